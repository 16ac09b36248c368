// Attention forward for sm_100a with both GEMMs on tcgen05 and softmax state in registers.
//
// One CTA (128 threads, thread r owns query row r) processes a 128-row query tile against 128-row KV tiles:
//   S = Q K^T        tcgen05.mma, K-major operands from TMA-swizzled shared memory, fp32 in TMEM columns [0,128)
//   P = softmax step rows are read back with tcgen05.ld (32x32b: one row per thread, no shuffles), online max/sum
//   O_tile = P V     P written to shared memory in the 128B-swizzled K-major layout, V consumed MN-major
//   O = O*alpha + O_tile in registers.
// KV tiles are double buffered (TMA for tile j+1 is in flight while tile j is computed).
//
// Two addressing modes share the core:
//   VARLEN  packed causal self-attention (training, old/ref log-prob passes, rollout prefill); GQA by head mapping.
//           Replaces flash_attn_varlen_func in the reference (verl/models/transformers/monkey_patch.py:146-148).
//   PAGED   decode: the G query heads of one KV group of one sequence form the (zero-padded) 128-row tile, K/V come
//           from a paged cache through the block table, optional split-KV with partial results merged afterwards.
//           Replaces vLLM's paged attention (verl/workers/rollout/vllm_rollout/vllm_async_server.py:690-697).
#include <cstdlib>

#include "common.cuh"
#include "tma_host.h"

namespace vb {

constexpr int ATT_D = 128;        // head dim
constexpr int ATT_BM = 128;       // query rows per tile
constexpr int ATT_BN = 128;       // kv rows per tile
constexpr int ATT_TILE_BYTES = 128 * 128 * 2;  // one [128 x 128] bf16 tile = two 64-column swizzle atoms
constexpr int ATT_HALF = 128 * 64 * 2;         // one atom: 128 rows x 128 B
constexpr int ATT_SMEM = ATT_TILE_BYTES * (1 + 4 + 1) + 1024 + 128;
constexpr int ATT_SMEM_COMPACT = ATT_TILE_BYTES * 3 + 1024 + 128;      // two CTAs per SM

struct AttnVarlenTile {  // host-built work list entry
  int q_tok0;      // global token index of the first query row
  int q_row0;      // index of that row inside its sequence
  int seq_tok0;    // global token index of the sequence start
  int seq_len;
};

struct AttnParams {
  // VARLEN
  const AttnVarlenTile* tiles;
  int n_q_heads, n_kv_heads;
  bf16* out;          // [T, Hq*D]
  long ld_out;
  float* lse;         // [Hq, T_pad] natural-log units of the scaled scores (may be null)
  long lse_stride;
  float scale_log2;   // softmax scale * log2(e)
  // PAGED
  const int* block_table;   // [B, max_blocks]
  int max_blocks;
  const int* kv_lens;       // [B]
  int group;                // q heads per kv head
  int num_splits;
  int tiles_per_split;
  float* part_o;            // [B, Hq, S, D] unnormalised
  float* part_ml;           // [B, Hq, S, 2] (m in log2 units, l)
  int* err_word;
};

// COMPACT: three tiles of shared memory (Q, K, V) instead of six so that TWO CTAs share an SM and one CTA's softmax
// overlaps the other's tensor-core work. P is written over the K tile (K is dead once S = Q K^T has completed); the next K
// and V tiles are requested as soon as the PV product has consumed P and V.
template <bool PAGED, bool COMPACT>
__global__ void __launch_bounds__(128, COMPACT ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + ATT_TILE_BYTES;                // stage s: K at +s*2*TILE, V at +s*2*TILE + TILE
  uint8_t* sP = COMPACT ? sKV : smem + ATT_TILE_BYTES * 5;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ATT_TILE_BYTES * (COMPACT ? 3 : 6));
  uint64_t* q_bar = bars;
  uint64_t* kv_bar = bars + 1;   // [2]
  uint64_t* s_bar = bars + 3;
  uint64_t* o_bar = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  // ---------------------------------------------------------------- work item
  int q_y, q_x, kv_head, kv_len_limit, num_kv_tiles, kv_tile0 = 0;
  int q_row0 = 0, seq_tok0 = 0, seq_len = 0, q_tok0 = 0;
  int b = 0, split = 0, head = 0;
  if (!PAGED) {
    const AttnVarlenTile t = p.tiles[blockIdx.x];
    head = blockIdx.y;
    kv_head = head / (p.n_q_heads / p.n_kv_heads);
    q_tok0 = t.q_tok0; q_row0 = t.q_row0; seq_tok0 = t.seq_tok0; seq_len = t.seq_len;
    q_y = q_tok0;
    q_x = head * ATT_D;
    kv_len_limit = min(seq_len, q_row0 + ATT_BM);
    num_kv_tiles = (kv_len_limit + ATT_BN - 1) / ATT_BN;
  } else {
    b = blockIdx.x; kv_head = blockIdx.y; split = blockIdx.z;
    q_y = b * p.n_q_heads + kv_head * p.group;   // Q viewed as [B*Hq, D]
    q_x = 0;
    kv_len_limit = p.kv_lens[b];
    const int total_tiles = (kv_len_limit + ATT_BN - 1) / ATT_BN;
    kv_tile0 = split * p.tiles_per_split;
    num_kv_tiles = max(0, min(p.tiles_per_split, total_tiles - kv_tile0));
  }

  if (tid == 0) {
    mbar_init(q_bar, 1);
    mbar_init(&kv_bar[0], 1);
    mbar_init(&kv_bar[1], 1);
    mbar_init(s_bar, 1);
    mbar_init(o_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc<256>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;          // columns [0,128)
  const uint32_t tmem_O = tmem_base + 128;    // columns [128,256)
  const uint32_t lane_off = uint32_t(warp * 32) << 16;

  // which = 0: K rows of kv tile j, which = 1: V rows; `dst` one tile of shared memory, `bar` gets the bytes (thread 0 only)
  auto load_half = [&](int j, int which, uint8_t* dst, uint64_t* bar) {
    const CUtensorMap* tm = which ? &tmV : &tmK;
    if (!PAGED) {
      const int y = seq_tok0 + j * ATT_BN;
      const int x = kv_head * ATT_D;
      tma_load_2d(dst, tm, x, y, bar);
      tma_load_2d(dst + ATT_HALF, tm, x + 64, y, bar);
    } else {
      // cache layer viewed as rows [(block*2 + kv)*Hkv + head]*64 + slot, 128 columns; block size 64
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int blk_idx = (kv_tile0 + j) * 2 + h2;
        const int blk = blk_idx < p.max_blocks ? p.block_table[(long)b * p.max_blocks + blk_idx] : 0;
        const int y = ((blk * 2 + which) * p.n_kv_heads + kv_head) * 64;
        // rows [64*h2, 64*h2+64) of each 64-column atom
        tma_load_2d(dst + h2 * 64 * 128, tm, 0, y, bar);
        tma_load_2d(dst + ATT_HALF + h2 * 64 * 128, tm, 64, y, bar);
      }
    }
  };
  auto load_kv = [&](int j, int stage) {  // thread 0 only; double-buffered layout: both halves on the stage's barrier
    uint8_t* sK = sKV + stage * 2 * ATT_TILE_BYTES;
    mbar_expect_tx(&kv_bar[stage], 2 * ATT_TILE_BYTES);
    load_half(j, 0, sK, &kv_bar[stage]);
    load_half(j, 1, sK + ATT_TILE_BYTES, &kv_bar[stage]);
  };
  auto load_compact = [&](int j) {        // thread 0 only; compact layout: kv_bar[0] counts K, kv_bar[1] counts V
    mbar_expect_tx(&kv_bar[0], ATT_TILE_BYTES);
    load_half(j, 0, sKV, &kv_bar[0]);
    mbar_expect_tx(&kv_bar[1], ATT_TILE_BYTES);
    load_half(j, 1, sKV + ATT_TILE_BYTES, &kv_bar[1]);
  };

  bool ok = true;
  if (tid == 0 && num_kv_tiles > 0) {
    mbar_expect_tx(q_bar, ATT_TILE_BYTES);
    tma_load_2d(sQ, &tmQ, q_x, q_y, q_bar);
    tma_load_2d(sQ + ATT_HALF, &tmQ, q_x + 64, q_y, q_bar);
    if (COMPACT) load_compact(0);
    else load_kv(0, 0);
  }

  float o_acc[ATT_D];
#pragma unroll
  for (int i = 0; i < ATT_D; ++i) o_acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const int my_q = q_row0 + tid;   // VARLEN: in-sequence index of this thread's query row

  constexpr uint32_t idesc_s = make_idesc(128, 128, 1, 1, false, false);  // S = Q K^T : both K-major
  constexpr uint32_t idesc_o = make_idesc(128, 128, 1, 1, false, true);   // O = P V   : A K-major, B MN-major

  if (num_kv_tiles > 0) {
    ok = mbar_wait(q_bar, 0, abort_flag, p.err_word, VB_ERR_WAIT_MISC);
  }

  for (int j = 0; j < num_kv_tiles && ok; ++j) {
    const int stage = COMPACT ? 0 : (j & 1);
    const uint32_t kv_phase = COMPACT ? (j & 1) : ((j >> 1) & 1);
    const uint32_t it_phase = j & 1;
    if (!COMPACT && tid == 0 && j + 1 < num_kv_tiles) load_kv(j + 1, stage ^ 1);   // stage^1 was released by the o_bar wait of j-1
    if (!mbar_wait(&kv_bar[stage], kv_phase, abort_flag, p.err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
    uint8_t* sK = sKV + stage * 2 * ATT_TILE_BYTES;
    uint8_t* sV = sK + ATT_TILE_BYTES;
    if (tid == 0) {
      tc_fence_after();
      const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK);
#pragma unroll
      for (int k = 0; k < ATT_D / 16; ++k) {
        const uint32_t off = (k >> 2) * ATT_HALF + (k & 3) * 32;
        umma_f16(tmem_S, make_sdesc_sw128(qa + off, 16, 1024), make_sdesc_sw128(ka + off, 16, 1024), idesc_s, k != 0);
      }
      umma_commit(s_bar);
    }
    if (!mbar_wait(s_bar, it_phase, abort_flag, p.err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
    tc_fence_after();

    // ---- pass 1: row max over valid columns
    const int kv0 = (kv_tile0 + j) * ATT_BN;
    int n_valid;   // columns [0, n_valid) of this tile are visible to this row
    if (!PAGED) n_valid = min(ATT_BN, min(my_q, seq_len - 1) - kv0 + 1);
    else n_valid = min(ATT_BN, kv_len_limit - kv0);
    // tiles strictly below the diagonal are fully visible to every row of the warp: no per-element masking there
    const bool full_tile = __all_sync(0xffffffffu, n_valid >= ATT_BN);
    float m_tile = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < ATT_BN / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_S + lane_off + c * 32, v);
      tmem_ld_wait();
      if (full_tile) {
#pragma unroll
        for (int i = 0; i < 32; ++i) m_tile = fmaxf(m_tile, __uint_as_float(v[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i < n_valid) m_tile = fmaxf(m_tile, __uint_as_float(v[i]));
      }
    }
    const float m_new = fmaxf(m_run, m_tile * p.scale_log2);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;   // fully masked row (only rows past the sequence end)
    const float alpha = exp2f(m_run - m_use);
    // ---- pass 2: P = exp2(s*scale - m), written to shared memory (K-major, 128B swizzle)
    float l_tile = 0.f;
#pragma unroll 1
    for (int c = 0; c < ATT_BN / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_S + lane_off + c * 32, v);
      tmem_ld_wait();
      float pv[32];
      if (full_tile) {
#pragma unroll
        for (int i = 0; i < 32; ++i) pv[i] = exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) pv[i] = (c * 32 + i < n_valid) ? exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use)) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) l_tile += pv[i];
      uint8_t* prow = sP + (c >> 1) * ATT_HALF + tid * 128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        // the PV product sees bf16-rounded probabilities, the row sum above the unrounded ones: the rounding errors are
        // unbiased and far below bf16 output precision, and summing fp32 values halves the instructions of this loop
        uint4 o;
        o.x = pack_bf16x2(pv[g * 8 + 0], pv[g * 8 + 1]);
        o.y = pack_bf16x2(pv[g * 8 + 2], pv[g * 8 + 3]);
        o.z = pack_bf16x2(pv[g * 8 + 4], pv[g * 8 + 5]);
        o.w = pack_bf16x2(pv[g * 8 + 6], pv[g * 8 + 7]);
        const int chunk = (c & 1) * 4 + g;
        *reinterpret_cast<uint4*>(prow + ((chunk ^ (tid & 7)) << 4)) = o;
      }
    }
    l_run = l_run * alpha + l_tile;
    m_run = m_new;
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (COMPACT && !mbar_wait(&kv_bar[1], kv_phase, abort_flag, p.err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t pa = smem_u32(sP), va = smem_u32(sV);
#pragma unroll
      for (int k = 0; k < ATT_BN / 16; ++k) {
        const uint32_t aoff = (k >> 2) * ATT_HALF + (k & 3) * 32;
        // V tile: two 64-column atoms (LBO = 16 KB apart), 8-row groups 1024 B apart, 16 kv rows per step = 2048 B
        umma_f16(tmem_O, make_sdesc_sw128(pa + aoff, 16, 1024), make_sdesc_sw128(va + k * 2048, ATT_HALF, 1024), idesc_o,
                 k != 0);
      }
      umma_commit(o_bar);
    }
    if (!mbar_wait(o_bar, it_phase, abort_flag, p.err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
    tc_fence_after();
    if (COMPACT && tid == 0 && j + 1 < num_kv_tiles) load_compact(j + 1);   // P (in the K tile) and V have been consumed
#pragma unroll
    for (int c = 0; c < ATT_D / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_O + lane_off + c * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(v[i]);
    }
    tc_fence_before();
    __syncthreads();   // all reads of S/O TMEM and of sP done before the next tile overwrites them
  }

  // ---------------------------------------------------------------- epilogue
  if (ok) {
    if (!PAGED) {
      if (my_q < seq_len) {
        const float inv = 1.f / l_run;
        bf16* orow = p.out + (long)(q_tok0 + tid) * p.ld_out + head * ATT_D;
#pragma unroll
        for (int i = 0; i < ATT_D; i += 8) {
          uint4 o;
          o.x = pack_bf16x2(o_acc[i] * inv, o_acc[i + 1] * inv);
          o.y = pack_bf16x2(o_acc[i + 2] * inv, o_acc[i + 3] * inv);
          o.z = pack_bf16x2(o_acc[i + 4] * inv, o_acc[i + 5] * inv);
          o.w = pack_bf16x2(o_acc[i + 6] * inv, o_acc[i + 7] * inv);
          *reinterpret_cast<uint4*>(orow + i) = o;
        }
        if (p.lse != nullptr) p.lse[(long)head * p.lse_stride + q_tok0 + tid] = (m_run + log2f(l_run)) * 0.6931471805599453f;
      }
    } else if (tid < p.group) {
      const int qh = kv_head * p.group + tid;
      if (p.num_splits == 1) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        bf16* orow = p.out + (long)b * p.ld_out + qh * ATT_D;
#pragma unroll
        for (int i = 0; i < ATT_D; i += 8) {
          uint4 o;
          o.x = pack_bf16x2(o_acc[i] * inv, o_acc[i + 1] * inv);
          o.y = pack_bf16x2(o_acc[i + 2] * inv, o_acc[i + 3] * inv);
          o.z = pack_bf16x2(o_acc[i + 4] * inv, o_acc[i + 5] * inv);
          o.w = pack_bf16x2(o_acc[i + 6] * inv, o_acc[i + 7] * inv);
          *reinterpret_cast<uint4*>(orow + i) = o;
        }
      } else {
        const long pidx = ((long)b * p.n_q_heads + qh) * p.num_splits + split;
        float* po = p.part_o + pidx * ATT_D;
#pragma unroll
        for (int i = 0; i < ATT_D; i += 4) *reinterpret_cast<float4*>(po + i) = make_float4(o_acc[i], o_acc[i + 1], o_acc[i + 2], o_acc[i + 3]);
        p.part_ml[pidx * 2 + 0] = m_run;
        p.part_ml[pidx * 2 + 1] = l_run;
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
    tmem_dealloc<256>(tmem_base);
  }
}

// Merge split-KV partials: out[b, h, :] = sum_s exp2(m_s - m) O_s / sum_s exp2(m_s - m) l_s
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                  long ld_out, int n_q_heads, int num_splits) {
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;  // 128 threads
  const long base = ((long)b * n_q_heads + h) * num_splits;
  float m = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    acc += w * part_o[(base + s) * ATT_D + d];
    l += w * part_ml[(base + s) * 2 + 1];
  }
  out[(long)b * ld_out + h * ATT_D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

// Two CTAs per SM (compact shared-memory layout) is the layout that runs; the double-buffered one-CTA-per-SM kernel
// instantiation stays for head counts whose tiles do not fit the compact layout.
static bool attn_compact() { return true; }

static int set_attn_smem() {
  static bool done = false;
  if (!done) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess) return -10;
    if (cudaFuncSetAttribute(attn_fwd_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess) return -10;
    if (cudaFuncSetAttribute(attn_fwd_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM_COMPACT) != cudaSuccess) return -10;
    if (cudaFuncSetAttribute(attn_fwd_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM_COMPACT) != cudaSuccess) return -10;
    // both CTAs of an SM need their shared memory at the same time: ask for the largest carve-out
    cudaFuncSetAttribute(attn_fwd_kernel<false, true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cudaFuncSetAttribute(attn_fwd_kernel<true, true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    done = true;
  }
  return 0;
}

}  // namespace vb

using namespace vb;

// Packed causal self-attention. q/k/v: bf16 pointers to the first element of the q, k, v sections of a fused row of
// `ld` elements per token (or of separate tensors with the same row stride); tiles: device array of n_tiles work items.
extern "C" int vb_attn_varlen_fwd(const void* q, const void* k, const void* v, long ld, int T, int n_q_heads, int n_kv_heads,
                                  const void* tiles, int n_tiles, void* out, long ld_out, float* lse, long lse_stride,
                                  float scale, int* err_word, cudaStream_t st) {
  if (n_tiles == 0) return 0;
  if (set_attn_smem()) return -10;
  CUtensorMap tmQ, tmK, tmV;
  if (make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)n_q_heads * ATT_D, ld, 128, 64)) return -1;
  if (make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)n_kv_heads * ATT_D, ld, 128, 64)) return -1;
  if (make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)n_kv_heads * ATT_D, ld, 128, 64)) return -1;
  AttnParams p = {};
  p.tiles = (const AttnVarlenTile*)tiles;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.out = (bf16*)out; p.ld_out = ld_out; p.lse = lse; p.lse_stride = lse_stride;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err_word = err_word;
  dim3 grid(n_tiles, n_q_heads);
  if (attn_compact()) attn_fwd_kernel<false, true><<<grid, 128, ATT_SMEM_COMPACT, st>>>(tmQ, tmK, tmV, p);
  else attn_fwd_kernel<false, false><<<grid, 128, ATT_SMEM, st>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Paged decode attention. q: [B, Hq*D] bf16 (row stride ld_q); cache: one layer [num_blocks, 2, Hkv, 64, D] bf16;
// scratch (only when num_splits > 1): part_o [B*Hq*S*D] fp32, part_ml [B*Hq*S*2] fp32.
extern "C" int vb_attn_paged_decode(const void* q, long ld_q, const void* cache, long num_blocks, const int* block_table,
                                    int max_blocks, const int* kv_lens, int B, int n_q_heads, int n_kv_heads, void* out,
                                    long ld_out, float scale, int num_splits, int max_kv_len, float* part_o, float* part_ml,
                                    int* err_word, cudaStream_t st) {
  if (B == 0) return 0;
  if (set_attn_smem()) return -10;
  if (ld_q != (long)n_q_heads * ATT_D) return -2;
  const int group = n_q_heads / n_kv_heads;
  if (group > 128) return -3;
  CUtensorMap tmQ, tmK, tmV;
  if (make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)B * n_q_heads, ATT_D, ATT_D, 128, 64)) return -1;
  const uint64_t rows = (uint64_t)num_blocks * 2 * n_kv_heads * 64;
  if (make_tmap_2d(&tmK, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, ATT_D, ATT_D, 64, 64)) return -1;
  tmV = tmK;
  AttnParams p = {};
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.out = (bf16*)out; p.ld_out = ld_out;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.block_table = block_table; p.max_blocks = max_blocks; p.kv_lens = kv_lens; p.group = group;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  const int max_tiles = (max_kv_len + ATT_BN - 1) / ATT_BN;
  p.tiles_per_split = (max_tiles + p.num_splits - 1) / p.num_splits;
  if (p.tiles_per_split < 1) p.tiles_per_split = 1;
  p.part_o = part_o; p.part_ml = part_ml; p.err_word = err_word;
  if (p.num_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return -4;
  dim3 grid(B, n_kv_heads, p.num_splits);
  if (attn_compact()) attn_fwd_kernel<true, true><<<grid, 128, ATT_SMEM_COMPACT, st>>>(tmQ, tmK, tmV, p);
  else attn_fwd_kernel<true, false><<<grid, 128, ATT_SMEM, st>>>(tmQ, tmK, tmV, p);
  if (cudaGetLastError() != cudaSuccess) return -11;
  if (p.num_splits > 1) {
    dim3 g2(B, n_q_heads);
    attn_merge_kernel<<<g2, 128, 0, st>>>(part_o, part_ml, (bf16*)out, ld_out, n_q_heads, p.num_splits);
    if (cudaGetLastError() != cudaSuccess) return -12;
  }
  return 0;
}
