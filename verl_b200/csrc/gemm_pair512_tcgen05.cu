// bf16 GEMM on SM pairs with 256 x 512 output tiles: the training-sized kernel.
//
// Why this shape. A 256 x 256 pair tile streams (256 + 256) operand rows per K step for 2*256*256 FLOPs per row pair;
// a 256 x 512 tile streams (256 + 512) rows for twice the FLOPs, i.e. 25 % fewer bytes from L2 into shared memory per
// FLOP. On a part that runs dense GEMMs at its power limit those bytes are clock: measured on B200 at 8192 x 37888 x
// 3584, the 256 x 256 kernel moved 1.34x the L2->SM bytes and 2.5x the DRAM bytes of the library kernel and ran at
// 1308 MHz against the library's 1460 MHz. The accumulator of one tile fills all 512 TMEM columns of both SMs, so tiles do
// not double-buffer in TMEM; instead the two 256-column halves are handed over separately (the MMA thread starts the next
// tile's first half while the epilogue still drains the second).
//
// Layout of a pair (cluster rank r = 0 "leader", r = 1 "peer"), per pipeline stage of one 64-element K block:
//   shared memory per CTA : A[128 x 64] rows m0 + 128 r | B0[128 x 64] columns n0 + 128 r | B1[128 x 64] columns n0 + 256 + 128 r
//   TMEM per CTA          : rows m0 + 128 r, 512 fp32 columns = half 0 (n0 .. n0+255) | half 1 (n0+256 .. n0+511)
//   MMA (leader thread)   : per K block, for each half h: four 256 x 256 x 16 tcgen05.mma.cta_group::2 into columns 256 h
// Epilogue: the four epilogue warps of each CTA read their 32 TMEM lanes 64 (bf16 out) or 32 (fp32 out) columns at a time,
// convert, stage the 32 x 128-byte slab in shared memory (128-byte swizzle, conflict-free, two buffers per warp) and hand it
// to the TMA unit (eight warps with one buffer each, four per half, measured no faster):
// a tiled store for bf16 / fp32 outputs, a tiled fp32 REDUCE-ADD when the GEMM accumulates into its output (weight
// gradients summed into the fp32 gradient buffer) — the addition happens at L2, nothing is read back into the SM.
// Edges need no code: out-of-range operand rows load as zeros and out-of-range output elements are clipped by the TMA unit.
//
// K slices: a GEMM that accumulates into an fp32 output may be cut along K into `split_k` slices per tile — every slice
// reduce-adds its partial tile, so no workspace and no second pass are needed. It is used when the tiles alone would leave
// the last wave of SM pairs mostly idle (weight gradients of the square projections: 98 tiles on 74 pairs).
//
// Tile order: row blocks are grouped so that one group's A panel (G x 256 x K) stays in L2 (about 28 MB) while the B
// panels stream past it once per group.
//
// Every wait is bounded (status word + normal teardown), as in the other kernels of this library.
#include "common.cuh"
#include "pair_common.cuh"
#include "tma_host.h"

namespace vb {
namespace pair512 {

using namespace vb::pair;

constexpr int BM = 128;                  // rows per CTA; a pair covers 256
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int HALF_N = 256;              // columns per MMA instruction / accumulator half
constexpr int TILE_N = 2 * HALF_N;
constexpr int A_TILE_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_HALF_BYTES = (HALF_N / 2) * BK * 2;  // this CTA's 128 rows of one half: 16 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + 2 * B_HALF_BYTES;   // 48 KB
constexpr int STAGES = 4;
constexpr int EPI_SLAB_BYTES = 32 * 128;             // 32 rows x 128 bytes
constexpr int EPI_WARPS = 4;
constexpr int EPI_BYTES = EPI_WARPS * 2 * EPI_SLAB_BYTES;   // two slab buffers per epilogue warp
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;

enum : int { FLAG_ACCUM = 1 };

__device__ __forceinline__ void tma_store_2d_tile(const CUtensorMap* m, uint32_t smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(reinterpret_cast<uint64_t>(m)),
               "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d_tile(const CUtensorMap* m, uint32_t smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair512_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
                    const bf16* __restrict__ bias, int M, int N, int K, int flags, int group_m, int split_k, int kb_per_split, int* err_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;                                       // 1024-byte aligned (48 KB stages)
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_smem + EPI_BYTES);              // used in the leader only
  uint64_t* empty_bar = full_bar + STAGES;                                               // one set per CTA
  uint64_t* tfull_bar = empty_bar + STAGES;                                              // one per CTA: the tile's accumulators are complete
  uint64_t* tempty_bar = tfull_bar + 1;                                                  // two (one per half), used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_n = (N + TILE_N - 1) / TILE_N;
  const int num_kb_total = (K + BK - 1) / BK;
  const int num_tiles = num_m * num_n * split_k;       // work units: (tile, K slice)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 2);      // one arrive.expect_tx from each CTA's producer
      mbar_init(&empty_bar[s], 1);     // one commit from the leader's MMA thread
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tempty_bar[0], 8);      // one arrival per epilogue warp of both CTAs
    mbar_init(&tempty_bar[1], 8);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair<TMEM_COLS>(tmem_slot);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                  // barriers of both CTAs exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto k_range = [&](int u, int& kb0, int& kb1) {
    kb0 = (u % split_k) * kb_per_split;
    kb1 = min(num_kb_total, kb0 + kb_per_split);
  };
  auto tile_coords = [&](int u, int& mb, int& nb) {
    const int t = u / split_k;
    const int per_group = group_m * num_n;
    const int g = t / per_group;
    const int first_m = g * group_m;
    const int gsz = min(num_m - first_m, group_m);
    const int r = t - g * per_group;
    mb = first_m + (r % gsz);
    nb = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        int mb, nb;
        tile_coords(t, mb, nb);
        const int m0 = mb * 2 * BM + (int)rank * BM;
        const int n0 = nb * TILE_N + (int)rank * (HALF_N / 2);
        int kb0, kb1;
        k_range(t, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, err_word, VB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[s]), 0);
          mbar_arrive_expect_tx_cluster(full_leader, STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmA, k0, m0, full_leader);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * (BK * 128), &tmA, m0 + 64 * i, k0, full_leader);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint8_t* sbh = sb + h * B_HALF_BYTES;
            const int nh = n0 + h * HALF_N;
            if (!B_MN) {
              tma_load_2d_pair(sbh, &tmB, k0, nh, full_leader);
            } else {
#pragma unroll
              for (int i = 0; i < (HALF_N / 2) / 64; ++i) tma_load_2d_pair(sbh + i * (BK * 128), &tmB, nh + 64 * i, k0, full_leader);
            }
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(2 * BM, HALF_N, 1, 1, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0, it = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs, ++it) {
        const uint32_t tph = it & 1;
        int kb0, kb1;
        k_range(t, kb0, kb1);
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (kb == kb0) {
              // the epilogue of the previous tile must have drained this half (first tile: passes at once)
              if (!mbar_wait(&tempty_bar[h], tph ^ 1, abort_flag, err_word, VB_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
              tc_fence_after();
            }
            const uint32_t sb = sa + A_TILE_BYTES + h * B_HALF_BYTES;
            const uint32_t d_tmem = tmem_base + h * HALF_N;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t ad = A_MN ? make_sdesc_sw128(sa + k * 2048, BK * 128, 1024) : make_sdesc_sw128(sa + k * 32, 16, 1024);
              const uint64_t bd = B_MN ? make_sdesc_sw128(sb + k * 2048, BK * 128, 1024) : make_sdesc_sw128(sb + k * 32, 16, 1024);
              umma_f16_pair(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0);
            }
          }
          if (!ok) break;
          const uint32_t e_local = smem_u32(&empty_bar[s]);
          umma_commit_pair(map_to_cta(e_local, 0));
          umma_commit_pair(map_to_cta(e_local, 1));
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) {
          const uint32_t f_local = smem_u32(&tfull_bar[0]);
          umma_commit_pair(map_to_cta(f_local, 0));
          umma_commit_pair(map_to_cta(f_local, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (four warps per CTA, 32 rows each)
    constexpr int CH = OUT_F32 ? 32 : 64;             // output columns per 128-byte slab row
    const int q = warp & 3;                           // TMEM lane quarter this warp may read
    const bool accum = flags & FLAG_ACCUM;
    uint8_t* slab_base = epi_smem + q * 2 * EPI_SLAB_BYTES;
    uint32_t it = 0, nslab = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs, ++it) {
      int mb, nb;
      tile_coords(t, mb, nb);
      const bool add_bias = bias != nullptr && (t % split_k) == 0;      // one K slice carries the bias
      if (lane == 0) ok = mbar_wait(&tfull_bar[0], it & 1, abort_flag, err_word, VB_ERR_WAIT_TMEM_FULL);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const int row0 = mb * 2 * BM + (int)rank * BM + q * 32;      // first row of this warp's slab
      const uint32_t lane_addr = tmem_base + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
#pragma unroll 1
        for (int c = 0; c < HALF_N / CH; ++c) {
          const int col0 = nb * TILE_N + h * HALF_N + c * CH;
          uint32_t v[64];
          tmem_ld_32x32b_x32(lane_addr + h * HALF_N + c * CH, v);
          if (!OUT_F32) tmem_ld_32x32b_x32(lane_addr + h * HALF_N + c * CH + 32, v + 32);
          tmem_ld_wait();
          if (add_bias) {
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (col0 + j < N) v[j] = __float_as_uint(__uint_as_float(v[j]) + __bfloat162float(bias[col0 + j]));
          }
          uint8_t* slab = slab_base + (nslab & 1) * EPI_SLAB_BYTES;
          ++nslab;
          // the TMA store that last read this slab buffer (two slabs ago) must be done reading it
          if (lane == 0) bulk_wait_read_1();
          __syncwarp();
          // row `lane` of the slab: eight 16-byte chunks, chunk j stored at position j ^ (lane & 7) (128-byte swizzle)
          uint8_t* srow = slab + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o;
            if (OUT_F32) {
              o = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
              o.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            }
            *reinterpret_cast<uint4*>(srow + ((j ^ (lane & 7)) << 4)) = o;
          }
          fence_async_smem();          // generic-proxy writes of this thread become visible to the TMA unit
          __syncwarp();
          if (lane == 0) {
            if (row0 < M && col0 < N) {
              if (OUT_F32 && accum) tma_reduce_add_2d_tile(&tmC, smem_u32(slab), col0, row0);
              else tma_store_2d_tile(&tmC, smem_u32(slab), col0, row0);
            }
            bulk_commit();             // an empty group when nothing was issued keeps the wait arithmetic uniform
          }
        }
        // this half of the accumulator is free for the next tile
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[h]), 0));
      }
    }
    if (lane == 0) bulk_wait_all();    // outstanding stores complete before the CTA may exit
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // a wait was abandoned: let copies and MMAs that are still in flight land before the ring and TMEM go away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) { __nanosleep(1000); }
  }
  __syncthreads();
  cluster_sync_all();                  // the peer may still be signalling this CTA's barriers until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair<TMEM_COLS>(tmem_base);
  }
}

static int g_sms = 0;
static int sm_count() {
  if (g_sms == 0) {
    int dev;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sms;
}

template <bool A_MN, bool B_MN, bool OUT_F32>
static int launch(const void* A, const void* B, void* Cp, const void* bias, int M, int N, int K, int lda, int ldb, int ldc, int flags,
                  int* err_word, cudaStream_t stream) {
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if (!A_MN) rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  else       rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, HALF_N / 2, BK);
  else       rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc) return rc;
  if (OUT_F32) rc = make_tmap_2d(&tmC, Cp, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, 32);
  else         rc = make_tmap_2d(&tmC, Cp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 32, 64);
  if (rc) return rc;
  static bool attr_set = false;
  auto kern = gemm_pair512_kernel<A_MN, B_MN, OUT_F32>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -10;
    attr_set = true;
  }
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  const int tiles0 = num_m * ((N + TILE_N - 1) / TILE_N);
  const int all_pairs = sm_count() / 2;
  // K slices (only where every slice can reduce-add into the fp32 output): pick the count that fills the last wave best
  const int num_kb = (K + BK - 1) / BK;
  int split_k = 1;
  if (OUT_F32 && (flags & FLAG_ACCUM)) {
    double best = (double)tiles0 / (((tiles0 + all_pairs - 1) / all_pairs) * all_pairs);
    for (int sk = 2; sk <= 8 && num_kb / sk >= 16; ++sk) {
      const long u = (long)tiles0 * sk;
      const double eff = (double)u / (((u + all_pairs - 1) / all_pairs) * all_pairs) - 0.01 * (sk - 1);      // a slice costs one more epilogue
      if (eff > best + 0.02) { best = eff; split_k = sk; }
    }
  }
  int kb_per = (num_kb + split_k - 1) / split_k;
  split_k = (num_kb + kb_per - 1) / kb_per;            // no empty slices
  const int tiles = tiles0 * split_k;
  int pairs = all_pairs;
  if (tiles < pairs) pairs = tiles;
  // row blocks per group: the group's A panel (G x 256 rows x K) should stay resident in L2 while B streams past it
  const long panel_bytes = 2l * BM * (long)K * 2;
  int group_m = (int)((28l << 20) / (panel_bytes > 0 ? panel_bytes : 1));
  if (group_m < 1) group_m = 1;
  if (group_m > num_m) group_m = num_m;
  kern<<<2 * pairs, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmC, reinterpret_cast<const bf16*>(bias), M, N, K, flags, group_m, split_k, kb_per, err_word);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace pair512
}  // namespace vb

// 1 when vb_gemm_bf16_pair512 can run this problem: output base 16-byte aligned with a row pitch that is a multiple of
// 16 bytes (TMA store), bf16 outputs not accumulated into.
extern "C" int vb_gemm_pair512_ok(const void* C, int ldc, int out_f32, int accumulate) {
  if (reinterpret_cast<uintptr_t>(C) & 15) return 0;
  if (out_f32) return (ldc & 3) == 0;
  return (ldc & 7) == 0 && !accumulate;
}

// Same contract as vb_gemm_bf16_pair: C[M,N] (+)= op(A) op(B) (+ bias) with 256 x 512 tiles on SM pairs. `accumulate` is
// supported for fp32 outputs (reduce-add at L2); check vb_gemm_pair512_ok first.
extern "C" int vb_gemm_bf16_pair512(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc,
                                    int a_mn, int b_mn, int out_f32, int accumulate, int* err_word, cudaStream_t stream) {
  using namespace vb::pair512;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -4;
  if (!vb_gemm_pair512_ok(C, ldc, out_f32, accumulate)) return -4;
  const int flags = accumulate ? FLAG_ACCUM : 0;
#define VB_P512(AM, BMN)                                                                                                         \
  return out_f32 ? launch<AM, BMN, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream)                         \
                 : launch<AM, BMN, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream)
  if (!a_mn && !b_mn) { VB_P512(false, false); }
  if (!a_mn && b_mn) { VB_P512(false, true); }
  if (a_mn && b_mn) { VB_P512(true, true); }
  VB_P512(true, false);
#undef VB_P512
}
