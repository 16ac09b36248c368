// Paged GQA decode attention for sm_100a, transposed formulation.
//
// One decode token per sequence has only G = Hq/Hkv (<= 16) query rows per KV head, so instead of padding them to a
// 128-row query tile the products are transposed:
//   S^T[kv, q] = K[kv, :] . Q[q, :]        tcgen05.mma M = 128 KV rows (TMEM lanes), N = 16 query heads
//   O^T[d, q]  = sum_kv V[kv, d] P[q, kv]   tcgen05.mma M = 128 head dims (V consumed MN-major), N = 16
// Every thread owns one KV row (softmax numerators) resp. one head-dim row (output) and touches 16 values per tile;
// row max / sum over the KV axis are warp-shuffle + shared-memory reductions. K/V tiles (128 rows) are fetched by TMA
// straight from the paged cache via the block table; the kernel is small enough (75 KB shared memory, 64 TMEM columns)
// for three CTAs per SM, which is what overlaps loads with the MMA -> softmax -> MMA chain of each tile. The score
// accumulator is double-buffered in TMEM: QK^T of tile j+1 is issued right behind the PV product of tile j, so it runs while
// the threads fold tile j's output and its result is ready when the next iteration asks for it. Optional split-KV writes partials merged by
// attn_merge_kernel (same layout as the generic paged path).
#include "common.cuh"
#include "tma_host.h"

namespace vb {

constexpr int DD = 128;                 // head dim
constexpr int DT = 128;                 // kv rows per tile
constexpr int DQ = 16;                  // padded query heads per kv head
constexpr int D_TILE = DT * DD * 2;     // 32 KB
constexpr int D_HALF = DT * 64 * 2;     // 16 KB : one 64-column swizzle atom of a K/V tile
constexpr int D_STAGES = 1;             // one K and one V buffer per CTA: K(j+1) streams in during softmax + PV of tile j, V(j+1) during
                                        // QK^T + softmax of tile j+1; three CTAs share an SM and hide the rest of the TMA latency
constexpr int D_QBYTES = DQ * DD * 2;   // 4 KB : two atoms of 16 rows x 128 B
constexpr int D_SMEM = D_STAGES * 2 * D_TILE + 2 * D_QBYTES + 1024 + 512;

struct DecodeParams {
  const int* block_table;
  int max_blocks;
  const int* kv_lens;
  int n_q_heads, n_kv_heads, group;
  int num_splits, tiles_per_split;
  bf16* out;
  long ld_out;
  float* part_o;
  float* part_ml;
  float scale_log2;
  int* err_word;
};

__global__ void __launch_bounds__(128, 3)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKV = smem;                                  // stage s: K at s*2*TILE, V at +TILE
  uint8_t* sQ = smem + D_STAGES * 2 * D_TILE;
  uint8_t* sP = sQ + D_QBYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + D_QBYTES);
  uint64_t* q_bar = bars;
  uint64_t* k_bar = bars + 1;
  uint64_t* v_bar = bars + 2;
  uint64_t* s_bar = bars + 4;
  uint64_t* o_bar = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(tmem_slot + 4);  // [4 warps][16]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int kv_len = p.kv_lens[b];
  const int total_tiles = (kv_len + DT - 1) / DT;
  const int tile0 = split * p.tiles_per_split;
  const int n_tiles = max(0, min(p.tiles_per_split, total_tiles - tile0));

  if (tid == 0) {
    mbar_init(q_bar, 1);
    mbar_init(k_bar, 1);
    mbar_init(v_bar, 1);
    mbar_init(s_bar, 1);
    mbar_init(o_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc<64>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S0 = tmem_base, tm_O = tmem_base + 32;       // scores of even tiles at +0, of odd tiles at +16
  const uint32_t lane_off = uint32_t(warp * 32) << 16;

  // which = 0: K rows of tile j into sK, which = 1: V rows into sV (thread 0)
  auto load_half = [&](int j, int which) {
    uint8_t* dst = sKV + which * D_TILE;
    uint64_t* bar = which ? v_bar : k_bar;
    mbar_expect_tx(bar, D_TILE);
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int bi = (tile0 + j) * 2 + h2;
      const int blk = bi < p.max_blocks ? p.block_table[(long)b * p.max_blocks + bi] : 0;
      const int y = ((blk * 2 + which) * p.n_kv_heads + kvh) * 64;
      tma_load_2d(dst + h2 * 64 * 128, &tmKV, 0, y, bar);
      tma_load_2d(dst + D_HALF + h2 * 64 * 128, &tmKV, 64, y, bar);
    }
  };

  if (tid == 0 && n_tiles > 0) {
    mbar_expect_tx(q_bar, D_QBYTES);
    const int qy = b * p.n_q_heads + kvh * p.group;
    tma_load_2d(sQ, &tmQ, 0, qy, q_bar);
    tma_load_2d(sQ + DQ * 128, &tmQ, 64, qy, q_bar);
    load_half(0, 0);
    load_half(0, 1);
  }

  float m_run[DQ], l_run[DQ], o_acc[DQ];
#pragma unroll
  for (int q = 0; q < DQ; ++q) { m_run[q] = -INFINITY; l_run[q] = 0.f; o_acc[q] = 0.f; }

  constexpr uint32_t idesc_s = make_idesc(128, DQ, 1, 1, false, false);   // K (K-major) x Q (K-major)
  constexpr uint32_t idesc_o = make_idesc(128, DQ, 1, 1, true, false);    // V^T (MN-major) x P (K-major)

  bool ok = true;
  if (n_tiles > 0) ok = mbar_wait(q_bar, 0, abort_flag, p.err_word, VB_ERR_WAIT_MISC);

  // QK^T of tile j into score buffer j & 1 (thread 0; waits for the tile's K rows itself)
  auto issue_qk = [&](int j) -> bool {
    if (!mbar_wait(k_bar, j & 1, abort_flag, p.err_word, VB_ERR_WAIT_FULL)) return false;
    tc_fence_after();
    const uint32_t ka = smem_u32(sKV), qa = smem_u32(sQ);
    const uint32_t tm_S = tm_S0 + (j & 1) * 16;
#pragma unroll
    for (int k = 0; k < DD / 16; ++k) {
      umma_f16(tm_S, make_sdesc_sw128(ka + (k >> 2) * D_HALF + (k & 3) * 32, 16, 1024),
               make_sdesc_sw128(qa + (k >> 2) * (DQ * 128) + (k & 3) * 32, 16, 1024), idesc_s, k != 0);
    }
    umma_commit(s_bar);
    return true;
  };
  if (ok && n_tiles > 0 && tid == 0) {
    if (!issue_qk(0)) *abort_flag = 1;
  }

  for (int j = 0; j < n_tiles && ok; ++j) {
    const uint32_t it_ph = j & 1;
    uint8_t* sV = sKV + D_TILE;
    if (!mbar_wait(s_bar, it_ph, abort_flag, p.err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && j + 1 < n_tiles) load_half(j + 1, 0);        // the K buffer is free once QK^T has completed
    uint32_t sv[DQ];
    tmem_ld_32x32b_x16(tm_S0 + it_ph * 16 + lane_off, sv);
    tmem_ld_wait();
    const bool valid = (tile0 + j) * DT + tid < kv_len;
    float s[DQ];
#pragma unroll
    for (int q = 0; q < DQ; ++q) s[q] = valid ? __uint_as_float(sv[q]) * p.scale_log2 : -INFINITY;
    // ---- column max over the 128 kv rows
#pragma unroll
    for (int q = 0; q < DQ; ++q) {
      float v = warp_max(s[q]);
      if (lane == 0) red[warp * DQ + q] = v;
    }
    __syncthreads();
    float alpha[DQ];
#pragma unroll
    for (int q = 0; q < DQ; ++q) {
      const float mt = fmaxf(fmaxf(red[q], red[DQ + q]), fmaxf(red[2 * DQ + q], red[3 * DQ + q]));
      const float mn = fmaxf(m_run[q], mt);
      const float mu = (mn == -INFINITY) ? 0.f : mn;
      alpha[q] = exp2f(m_run[q] - mu);
      m_run[q] = mn;
      s[q] = valid ? exp2f(s[q] - mu) : 0.f;              // s now holds the probability numerator
    }
    __syncthreads();                                       // everyone has read `red` before it is reused for the sums
    // ---- P (K-major [16 q rows x 128 kv cols], 128B swizzle): element (q, kv = tid)
    {
      uint8_t* pbase = sP + (tid >> 6) * (DQ * 128);
      const int c = tid & 63;
#pragma unroll
      for (int q = 0; q < DQ; ++q) {
        const __nv_bfloat16 pb = __float2bfloat16(s[q]);
        *reinterpret_cast<__nv_bfloat16*>(pbase + q * 128 + ((((c >> 3) ^ (q & 7))) << 4) + (c & 7) * 2) = pb;
        s[q] = __bfloat162float(pb);
      }
    }
#pragma unroll
    for (int q = 0; q < DQ; ++q) {
      float v = warp_sum(s[q]);
      if (lane == 0) red[warp * DQ + q] = v;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (!mbar_wait(v_bar, it_ph, abort_flag, p.err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t va = smem_u32(sV), pa = smem_u32(sP);
#pragma unroll
      for (int k = 0; k < DT / 16; ++k) {
        umma_f16(tm_O, make_sdesc_sw128(va + k * 2048, D_HALF, 1024),
                 make_sdesc_sw128(pa + (k >> 2) * (DQ * 128) + (k & 3) * 32, 16, 1024), idesc_o, k != 0);
      }
      umma_commit(o_bar);
      // the next tile's scores: its K rows were requested when this tile's QK^T had completed, and the other score buffer was
      // last read by the softmax of tile j-1
      if (j + 1 < n_tiles && !issue_qk(j + 1)) *abort_flag = 1;
    }
#pragma unroll
    for (int q = 0; q < DQ; ++q) l_run[q] = l_run[q] * alpha[q] + red[q] + red[DQ + q] + red[2 * DQ + q] + red[3 * DQ + q];
    if (!mbar_wait(o_bar, it_ph, abort_flag, p.err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && j + 1 < n_tiles) load_half(j + 1, 1);        // the V buffer is free once the PV product has completed
    uint32_t ov[DQ];
    tmem_ld_32x32b_x16(tm_O + lane_off, ov);
    tmem_ld_wait();
#pragma unroll
    for (int q = 0; q < DQ; ++q) o_acc[q] = o_acc[q] * alpha[q] + __uint_as_float(ov[q]);
    tc_fence_before();
    __syncthreads();
  }

  if (ok) {
    const int d = tid;   // this thread owns head-dim row d of O^T
    for (int q = 0; q < p.group; ++q) {
      const int qh = kvh * p.group + q;
      if (p.num_splits == 1) {
        const float inv = l_run[q] > 0.f ? 1.f / l_run[q] : 0.f;
        p.out[(long)b * p.ld_out + qh * DD + d] = __float2bfloat16(o_acc[q] * inv);
      } else {
        const long pidx = ((long)b * p.n_q_heads + qh) * p.num_splits + split;
        p.part_o[pidx * DD + d] = o_acc[q];
        if (d == 0) {
          p.part_ml[pidx * 2 + 0] = m_run[q];
          p.part_ml[pidx * 2 + 1] = l_run[q];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (*abort_flag) {
      uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) { __nanosleep(1000); }
    }
    tc_fence_after();
    tmem_dealloc<64>(tmem_base);
  }
}

__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                         long ld_out, int n_q_heads, int num_splits) {
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const long base = ((long)b * n_q_heads + h) * num_splits;
  float m = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    acc += w * part_o[(base + s) * DD + d];
    l += w * part_ml[(base + s) * 2 + 1];
  }
  out[(long)b * ld_out + h * DD + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace vb

using namespace vb;

// Same contract as vb_attn_paged_decode; requires Hq/Hkv <= 16.
extern "C" int vb_attn_decode_gqa(const void* q, long ld_q, const void* cache, long num_blocks, const int* block_table,
                                  int max_blocks, const int* kv_lens, int B, int n_q_heads, int n_kv_heads, void* out, long ld_out,
                                  float scale, int num_splits, int max_kv_len, float* part_o, float* part_ml, int* err_word,
                                  cudaStream_t st) {
  if (B == 0) return 0;
  const int group = n_q_heads / n_kv_heads;
  if (group > DQ) return -3;
  if (ld_q != (long)n_q_heads * DD) return -2;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, D_SMEM) != cudaSuccess) return -10;
    attr = true;
  }
  CUtensorMap tmQ, tmKV;
  if (make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * n_q_heads, DD, DD, DQ, 64)) return -1;
  const uint64_t rows = (uint64_t)num_blocks * 2 * n_kv_heads * 64;
  if (make_tmap_2d(&tmKV, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, DD, DD, 64, 64)) return -1;
  DecodeParams p = {};
  p.block_table = block_table; p.max_blocks = max_blocks; p.kv_lens = kv_lens;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.group = group;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  const int max_tiles = (max_kv_len + DT - 1) / DT;
  p.tiles_per_split = (max_tiles + p.num_splits - 1) / p.num_splits;
  if (p.tiles_per_split < 1) p.tiles_per_split = 1;
  p.out = (bf16*)out; p.ld_out = ld_out; p.part_o = part_o; p.part_ml = part_ml;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err_word = err_word;
  if (p.num_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return -4;
  dim3 grid(B, n_kv_heads, p.num_splits);
  attn_decode_kernel<<<grid, 128, D_SMEM, st>>>(tmQ, tmKV, p);
  if (cudaGetLastError() != cudaSuccess) return -11;
  if (p.num_splits > 1) {
    dim3 g2(B, n_q_heads);
    attn_decode_merge_kernel<<<g2, 128, 0, st>>>(part_o, part_ml, (bf16*)out, ld_out, n_q_heads, p.num_splits);
    if (cudaGetLastError() != cudaSuccess) return -12;
  }
  return 0;
}
