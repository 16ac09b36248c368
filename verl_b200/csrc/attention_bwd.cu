// Attention backward (packed causal varlen, GQA) for sm_100a: all five GEMMs on tcgen05.
//
// One CTA owns one 128-row KV tile of one sequence for one KV head and loops over the G query heads of the group and
// the query tiles at or below it (causal):
//   S  = Q K^T, dP = dO V^T            both into TMEM (lanes = query rows)
//   P  = exp2(S*c - lse), dS = P o (dP - delta) * scale   per-thread rows, written as bf16 to shared memory once;
//        the same swizzled [q, kv] buffer is the K-major A operand of dS*K and the MN-major A operand of P^T*dO, dS^T*Q
//   dV += P^T dO, dK += dS^T Q         accumulated in TMEM across all iterations (never leave the SM until the end)
//   dQ  = dS K                         into the (already consumed) S columns, then fp32 vector atomics to global
// Replaces flash-attn's backward used through transformers in the reference
// (verl/models/transformers/monkey_patch.py:146-148).
#include "common.cuh"
#include "tma_host.h"

namespace vb {

constexpr int AB_D = 128;
constexpr int AB_TILE = 128 * 128 * 2;
constexpr int AB_HALF = 128 * 64 * 2;
constexpr int AB_SMEM = AB_TILE * 6 + 1024 + 128;

struct AttnBwdTile {
  int kv_tok0;     // global token of first kv row of this tile
  int kv_row0;     // in-sequence index of that row (multiple of 128)
  int seq_tok0;
  int seq_len;
  int q_tile_begin;   // first 128-row query tile of the sequence that has real queries (context parallelism: the rows before
                      // it only carry keys/values); 0 for ordinary batches
  int pad[3];
};

struct AttnBwdParams {
  const AttnBwdTile* tiles;
  int n_q_heads, n_kv_heads;
  const float* lse;     // [Hq, stride] natural log
  const float* delta;   // [Hq, stride]
  long stat_stride;
  float* dq_acc;        // [T, Hq*D] fp32, zero-initialised
  bf16* dk;             // row stride ld_dkv, head offset applied inside
  bf16* dv;
  long ld_dkv;
  float scale;
  float scale_log2;
  int* err_word;
};

__global__ void __launch_bounds__(128, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + AB_TILE;
  uint8_t* sQ = smem + 2 * AB_TILE;
  uint8_t* sdO = smem + 3 * AB_TILE;
  uint8_t* sP = smem + 4 * AB_TILE;
  uint8_t* sdS = smem + 5 * AB_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * AB_TILE);
  uint64_t* kv_bar = bars;
  uint64_t* qdo_bar = bars + 1;
  uint64_t* s_bar = bars + 2;
  uint64_t* mma_bar = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const AttnBwdTile t = p.tiles[blockIdx.x];
  const int kv_head = blockIdx.y;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int n_q_tiles_total = (t.seq_len + 127) / 128;
  const int first_q_tile = max(t.kv_row0 / 128, t.q_tile_begin);
  const int iters_per_head = n_q_tiles_total - first_q_tile;
  const int n_iters = iters_per_head * group;

  if (tid == 0) {
    mbar_init(kv_bar, 1);
    mbar_init(qdo_bar, 1);
    mbar_init(s_bar, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc<512>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base;           // also receives dQ
  const uint32_t tm_dP = tmem_base + 128;
  const uint32_t tm_dV = tmem_base + 256;
  const uint32_t tm_dK = tmem_base + 384;
  const uint32_t lane_off = uint32_t(warp * 32) << 16;

  auto load_qdo = [&](int it) {  // thread 0
    const int hh = it / iters_per_head;
    const int qt = first_q_tile + (it - hh * iters_per_head);
    const int head = kv_head * group + hh;
    const int y = t.seq_tok0 + qt * 128;
    const int x = head * AB_D;
    mbar_expect_tx(qdo_bar, 2 * AB_TILE);
    tma_load_2d(sQ, &tmQ, x, y, qdo_bar);
    tma_load_2d(sQ + AB_HALF, &tmQ, x + 64, y, qdo_bar);
    tma_load_2d(sdO, &tmdO, x, y, qdo_bar);
    tma_load_2d(sdO + AB_HALF, &tmdO, x + 64, y, qdo_bar);
  };

  if (tid == 0) {
    mbar_expect_tx(kv_bar, 2 * AB_TILE);
    const int x = kv_head * AB_D;
    tma_load_2d(sK, &tmK, x, t.kv_tok0, kv_bar);
    tma_load_2d(sK + AB_HALF, &tmK, x + 64, t.kv_tok0, kv_bar);
    tma_load_2d(sV, &tmV, x, t.kv_tok0, kv_bar);
    tma_load_2d(sV + AB_HALF, &tmV, x + 64, t.kv_tok0, kv_bar);
    if (n_iters > 0) load_qdo(0);
  }
  bool ok = mbar_wait(kv_bar, 0, abort_flag, p.err_word, VB_ERR_WAIT_FULL);

  constexpr uint32_t idesc_kk = make_idesc(128, 128, 1, 1, false, false);  // K-major x K-major
  constexpr uint32_t idesc_mm = make_idesc(128, 128, 1, 1, true, true);    // MN-major A (transposed smem) x MN-major B
  constexpr uint32_t idesc_km = make_idesc(128, 128, 1, 1, false, true);   // K-major A x MN-major B

  for (int it = 0; it < n_iters && ok; ++it) {
    const uint32_t ph = it & 1;
    const int hh = it / iters_per_head;
    const int qt = first_q_tile + (it - hh * iters_per_head);
    const int head = kv_head * group + hh;
    const int q_row0 = qt * 128;
    if (!mbar_wait(qdo_bar, ph, abort_flag, p.err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK), da = smem_u32(sdO), va = smem_u32(sV);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t off = (k >> 2) * AB_HALF + (k & 3) * 32;
        umma_f16(tm_S, make_sdesc_sw128(qa + off, 16, 1024), make_sdesc_sw128(ka + off, 16, 1024), idesc_kk, k != 0);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t off = (k >> 2) * AB_HALF + (k & 3) * 32;
        umma_f16(tm_dP, make_sdesc_sw128(da + off, 16, 1024), make_sdesc_sw128(va + off, 16, 1024), idesc_kk, k != 0);
      }
      umma_commit(s_bar);
    }
    // per-row statistics while the MMAs run
    const int my_q = q_row0 + tid;
    const bool row_ok = my_q < t.seq_len;
    float lse2 = 0.f, dl = 0.f;
    if (row_ok) {
      const long si = (long)head * p.stat_stride + t.seq_tok0 + my_q;
      lse2 = p.lse[si] * 1.4426950408889634f;
      dl = p.delta[si];
    }
    const int n_valid = row_ok ? min(128, my_q - t.kv_row0 + 1) : 0;   // causal: kv index <= q index
    const bool full_tile = __all_sync(0xffffffffu, n_valid >= 128);
    if (!mbar_wait(s_bar, ph, abort_flag, p.err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t sv[32], dv[32];
      tmem_ld_32x32b_x32(tm_S + lane_off + c * 32, sv);
      tmem_ld_32x32b_x32(tm_dP + lane_off + c * 32, dv);
      tmem_ld_wait();
      uint8_t* prow = sP + (c >> 1) * AB_HALF + tid * 128;
      uint8_t* drow = sdS + (c >> 1) * AB_HALF + tid * 128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float pf[8], df[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int col = c * 32 + g * 8 + e;
          // query tiles strictly below the diagonal see the whole kv tile: no per-element mask there
          const float pe = (full_tile || col < n_valid) ? exp2f(fmaf(__uint_as_float(sv[g * 8 + e]), p.scale_log2, -lse2)) : 0.f;
          pf[e] = pe;
          df[e] = pe * (__uint_as_float(dv[g * 8 + e]) - dl) * p.scale;
        }
        uint4 po, dso;
        po.x = pack_bf16x2(pf[0], pf[1]); po.y = pack_bf16x2(pf[2], pf[3]);
        po.z = pack_bf16x2(pf[4], pf[5]); po.w = pack_bf16x2(pf[6], pf[7]);
        dso.x = pack_bf16x2(df[0], df[1]); dso.y = pack_bf16x2(df[2], df[3]);
        dso.z = pack_bf16x2(df[4], df[5]); dso.w = pack_bf16x2(df[6], df[7]);
        const int chunk = ((c & 1) * 4 + g) ^ (tid & 7);
        *reinterpret_cast<uint4*>(prow + (chunk << 4)) = po;
        *reinterpret_cast<uint4*>(drow + (chunk << 4)) = dso;
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t pa = smem_u32(sP), dsa = smem_u32(sdS), qa = smem_u32(sQ), da = smem_u32(sdO), ka = smem_u32(sK);
      // dV[kv,d] += P^T[kv,q] dO[q,d] ; dK[kv,d] += dS^T[kv,q] Q[q,d] : contraction over the 128 query rows
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        umma_f16(tm_dV, make_sdesc_sw128(pa + k * 2048, AB_HALF, 1024), make_sdesc_sw128(da + k * 2048, AB_HALF, 1024), idesc_mm,
                 (it | k) != 0);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        umma_f16(tm_dK, make_sdesc_sw128(dsa + k * 2048, AB_HALF, 1024), make_sdesc_sw128(qa + k * 2048, AB_HALF, 1024), idesc_mm,
                 (it | k) != 0);
      }
      // dQ[q,d] = dS[q,kv] K[kv,d] : contraction over the 128 kv rows; reuses the S columns
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t aoff = (k >> 2) * AB_HALF + (k & 3) * 32;
        umma_f16(tm_S, make_sdesc_sw128(dsa + aoff, 16, 1024), make_sdesc_sw128(ka + k * 2048, AB_HALF, 1024), idesc_km, k != 0);
      }
      umma_commit(mma_bar);
    }
    if (!mbar_wait(mma_bar, ph, abort_flag, p.err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && it + 1 < n_iters) load_qdo(it + 1);   // sQ / sdO are free now; overlaps the dQ read-out
    {
      // TMEM loads are warp-collective: every lane executes them; only in-sequence rows add to global memory
      float* dq = p.dq_acc + (long)(t.seq_tok0 + my_q) * ((long)p.n_q_heads * AB_D) + head * AB_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tm_S + lane_off + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 a = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            atomicAdd(reinterpret_cast<float4*>(dq + c * 32 + i), a);
          }
        }
      }
    }
    tc_fence_before();
    __syncthreads();
  }

  // ---------------------------------------------------------------- write dK, dV (lanes = kv rows)
  if (ok) {
    const int my_kv = t.kv_row0 + tid;
    const bool row_ok = my_kv < t.seq_len && n_iters > 0;
    bf16* dkrow = p.dk + (long)(t.kv_tok0 + tid) * p.ld_dkv + kv_head * AB_D;
    bf16* dvrow = p.dv + (long)(t.kv_tok0 + tid) * p.ld_dkv + kv_head * AB_D;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t a[32], b2[32];
      tmem_ld_32x32b_x32(tm_dK + lane_off + c * 32, a);
      tmem_ld_32x32b_x32(tm_dV + lane_off + c * 32, b2);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 o1, o2;
          o1.x = pack_bf16x2(__uint_as_float(a[i]), __uint_as_float(a[i + 1]));
          o1.y = pack_bf16x2(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
          o1.z = pack_bf16x2(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5]));
          o1.w = pack_bf16x2(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
          o2.x = pack_bf16x2(__uint_as_float(b2[i]), __uint_as_float(b2[i + 1]));
          o2.y = pack_bf16x2(__uint_as_float(b2[i + 2]), __uint_as_float(b2[i + 3]));
          o2.z = pack_bf16x2(__uint_as_float(b2[i + 4]), __uint_as_float(b2[i + 5]));
          o2.w = pack_bf16x2(__uint_as_float(b2[i + 6]), __uint_as_float(b2[i + 7]));
          *reinterpret_cast<uint4*>(dkrow + c * 32 + i) = o1;
          *reinterpret_cast<uint4*>(dvrow + c * 32 + i) = o2;
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
    tmem_dealloc<512>(tmem_base);
  }
}

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d] ; one warp per (t, h)
__global__ void attn_delta_kernel(const bf16* __restrict__ dO, const bf16* __restrict__ O, long ld, float* __restrict__ delta,
                                  long stride, int T, int H) {
  const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long)T * H) return;
  const int h = w % H;
  const long tk = w / H;
  const bf16* a = dO + tk * ld + h * AB_D + lane * 4;
  const bf16* b = O + tk * ld + h * AB_D + lane * 4;
  const uint2 av = *reinterpret_cast<const uint2*>(a);
  const uint2 bv = *reinterpret_cast<const uint2*>(b);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(b2[i]);
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(long)h * stride + tk] = s;
}

// dq bf16 section of the fused gradient row from the fp32 accumulator
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ out, long ld_out, long T, int cols) {
  const long n4 = T * cols / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    const long e = i * 4;
    const long tk = e / cols;
    const int c = e % cols;
    const float4 v = *reinterpret_cast<const float4*>(acc + e);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(out + tk * ld_out + c) = o;
  }
}

}  // namespace vb

using namespace vb;

// q/k/v/dO/O as in the forward; dq_acc: fp32 [T, Hq*D] scratch (zeroed here); dqkv sections dq/dk/dv share row stride ld_d.
extern "C" int vb_attn_varlen_bwd(const void* q, const void* k, const void* v, long ld, const void* dO, const void* O, long ld_o,
                                  int T, int n_q_heads, int n_kv_heads, const void* tiles, int n_tiles, const float* lse,
                                  float* delta, long stat_stride, float* dq_acc, void* dq, void* dk, void* dv, long ld_d,
                                  float scale, int* err_word, cudaStream_t st) {
  if (n_tiles == 0 || T == 0) return 0;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AB_SMEM) != cudaSuccess) return -10;
    attr = true;
  }
  CUtensorMap tmQ, tmK, tmV, tmdO;
  if (make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)n_q_heads * AB_D, ld, 128, 64)) return -1;
  if (make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)n_kv_heads * AB_D, ld, 128, 64)) return -1;
  if (make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)n_kv_heads * AB_D, ld, 128, 64)) return -1;
  if (make_tmap_2d(&tmdO, dO, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)n_q_heads * AB_D, ld_o, 128, 64)) return -1;
  {
    const long warps = (long)T * n_q_heads;
    const int block = 256;
    const long blocks = (warps * 32 + block - 1) / block;
    attn_delta_kernel<<<(unsigned)blocks, block, 0, st>>>((const bf16*)dO, (const bf16*)O, ld_o, delta, stat_stride, T, n_q_heads);
  }
  cudaMemsetAsync(dq_acc, 0, (size_t)T * n_q_heads * AB_D * sizeof(float), st);
  AttnBwdParams p = {};
  p.tiles = (const AttnBwdTile*)tiles;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.lse = lse; p.delta = delta; p.stat_stride = stat_stride;
  p.dq_acc = dq_acc; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.ld_dkv = ld_d;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.err_word = err_word;
  dim3 grid(n_tiles, n_kv_heads);
  attn_bwd_kernel<<<grid, 128, AB_SMEM, st>>>(tmQ, tmK, tmV, tmdO, p);
  if (cudaGetLastError() != cudaSuccess) return -11;
  const long n4 = (long)T * n_q_heads * AB_D / 4;
  int blocks = (int)((n4 + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  attn_dq_convert_kernel<<<blocks, 256, 0, st>>>(dq_acc, (bf16*)dq, ld_d, T, n_q_heads * AB_D);
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}
