// bf16 GEMM with two CTAs (one thread-block cluster of 2 = two SMs) cooperating on one 256 x BN output tile through
// tcgen05.mma.cta_group::2.
//
// Why: with a single-CTA 128x256 MMA every SM streams 128 rows of A and 256 rows of B from shared memory for each K
// step, which nearly saturates the shared-memory read path. In pair mode the two SMs each hold their own 128 rows of
// A but only HALF of the B tile (BN/2 rows); the tensor cores of both SMs read both halves, so per-SM operand
// traffic drops by a third and the same ring holds deeper pipelines.
//
// Layout of a pair (cluster rank r = 0 "leader", r = 1 "peer"):
//   * shared memory ring per CTA: A[128 x 64] of rows m0 + 128 r, B[(BN/2) x 64] of columns n0 + (BN/2) r;
//   * TMEM per CTA: accumulator rows m0 + 128 r .. +127, BN fp32 columns, double buffered;
//   * producer warp (each CTA): waits its own `empty`, announces its bytes on the LEADER's `full` barrier and issues
//     its TMA loads with the leader's barrier as completion target (cp.async.bulk.tensor ... cta_group::2);
//   * MMA thread (leader only): waits `full`, issues the 256-row MMAs, then commits to `empty` of BOTH CTAs;
//   * epilogue warps (each CTA): wait their own `tmem full`, read their own TMEM lanes, store their 128 rows, and
//     arrive on the leader's `tmem empty` barrier (count 256).
// Every wait is bounded; a pair that gives up records a status word and both CTAs still meet at the closing cluster
// barrier so neither exits while the other may touch its shared memory.
#include "common.cuh"
#include "pair_common.cuh"
#include "tma_host.h"

extern "C" int vb_splitk_reduce(const float* ws, int S, int M, int N, void* out, int ldc, const void* bias, int out_f32, int accumulate,
                                cudaStream_t stream);

namespace vb {
namespace pair {

constexpr int BM = 128;          // rows per CTA; a pair covers 256
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;

template <int BN>
struct Cfg {
  static constexpr int B_TILE_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int MAX_STAGES = (216 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN;
};

enum : int { OUT_F32 = 1, ACCUM = 2 };

// FP8: operands are e4m3 bytes, K-major; a stage row is still 128 bytes (128 elements of K instead of 64) so the ring, the
// swizzle and the descriptors are unchanged. The epilogue applies per-row (a_scale[M]) and per-column (b_scale[N]) scales.
template <int BN, bool A_MN, bool B_MN, bool FP8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cv,
                 const bf16* __restrict__ bias, int M, int N, int K, int ldc, int flags, int* err_word,
                 const float* __restrict__ a_scale, const float* __restrict__ b_scale, int split_k, int kb_per_split,
                 float* __restrict__ split_ws) {
  // split_k > 1: a work unit is (output tile, K slice); every slice stores its fp32 partial tile into
  // split_ws[slice][M][N] and a reduce pass (vb_splitk_reduce) adds them up, applies bias / accumulate and casts
  static_assert(!FP8 || (!A_MN && !B_MN), "fp8 operands are K-major");
  constexpr int BKE = FP8 ? 2 * BK : BK;      // elements of K per stage
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);   // used in the leader only
  uint64_t* empty_bar = full_bar + STAGES;                                              // one set per CTA
  uint64_t* tfull_bar = empty_bar + STAGES;                                             // one set per CTA
  uint64_t* tempty_bar = tfull_bar + 2;                                                 // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_n = (N + BN - 1) / BN;
  const int num_kb_total = (K + BKE - 1) / BKE;
  const int num_tiles = num_m * num_n * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 2);      // one arrive.expect_tx from each CTA's producer
      mbar_init(&empty_bar[s], 1);     // one commit from the leader's MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 256);  // the epilogue threads of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair<C::TMEM_COLS>(tmem_slot);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                  // barriers of both CTAs exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr int GROUP_M = 4;           // 4 x 256 rows share a B column block in L2
  auto k_range = [&](int u, int& kb0, int& kb1) {
    kb0 = (u % split_k) * kb_per_split;
    kb1 = min(num_kb_total, kb0 + kb_per_split);
  };
  auto tile_coords = [&](int u, int& mb, int& nb) {
    const int t = u / split_k;
    int per_group = GROUP_M * num_n;
    int g = t / per_group;
    int first_m = g * GROUP_M;
    int gsz = min(num_m - first_m, GROUP_M);
    int r = t - g * per_group;
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
        const int n0 = nb * BN + (int)rank * (BN / 2);
        int kb0, kb1;
        k_range(t, kb0, kb1);
        // few row blocks: stagger the K order per column block so the CTAs do not all ask for the same A tile at once
        const int nk = kb1 - kb0;
        const int rot = (num_m <= 2 && nk > 1) ? (nb * 5) % nk : 0;
        for (int ki = 0; ki < nk; ++ki) {
          const int kb = kb0 + (ki + rot >= nk ? ki + rot - nk : ki + rot);
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, err_word, VB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * C::STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[s]), 0);
          mbar_arrive_expect_tx_cluster(full_leader, C::STAGE_BYTES);
          const int k0 = kb * BKE;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmA, k0, m0, full_leader);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * (BK * 128), &tmA, m0 + 64 * i, k0, full_leader);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmB, k0, n0, full_leader);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 128; ++i) tma_load_2d_pair(sb + i * (BK * 128), &tmB, n0 + 64 * i, k0, full_leader);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = FP8 ? make_idesc(2 * BM, BN, 0, 0, false, false) : make_idesc(2 * BM, BN, 1, 1, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0, it = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs, ++it) {
        const uint32_t acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, err_word, VB_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int kb0, kb1;
        k_range(t, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = A_MN ? make_sdesc_sw128(sa + k * 2048, BK * 128, 1024) : make_sdesc_sw128(sa + k * 32, 16, 1024);
            uint64_t bd = B_MN ? make_sdesc_sw128(sb + k * 2048, BK * 128, 1024) : make_sdesc_sw128(sb + k * 32, 16, 1024);
            if constexpr (FP8) umma_f8_pair(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0);
            else umma_f16_pair(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0);
          }
          const uint32_t e_local = smem_u32(&empty_bar[s]);
          umma_commit_pair(map_to_cta(e_local, 0));
          umma_commit_pair(map_to_cta(e_local, 1));
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) {
          const uint32_t f_local = smem_u32(&tfull_bar[acc]);
          umma_commit_pair(map_to_cta(f_local, 0));
          umma_commit_pair(map_to_cta(f_local, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (128 threads per CTA, own rows)
    const int q = warp & 3;
    const bool out_f32 = flags & OUT_F32;
    const bool accum = flags & ACCUM;
    uint32_t it = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs, ++it) {
      int mb, nb;
      tile_coords(t, mb, nb);
      const uint32_t acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * 2 * BM + (int)rank * BM + q * 32 + lane;
      const int n0 = nb * BN;
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + c * 32, v);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (split_k > 1) {
            float* wrow = split_ws + ((size_t)(t % split_k) * M + row) * N + col0;
            if (col0 + 32 <= N) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(wrow + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) wrow[j] = f[j];
            }
            continue;
          }
          if constexpr (FP8) {
            if (a_scale != nullptr) {
              const float rs = a_scale[row];
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) f[j] *= rs * b_scale[col0 + j];
            }
          }
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) f[j] += __bfloat162float(bias[col0 + j]);
          }
          const bool full = (col0 + 32 <= N);
          if (out_f32) {
            float* crow = reinterpret_cast<float*>(Cv) + (size_t)row * ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
                if (accum) {
                  const float4 p = *reinterpret_cast<float4*>(crow + j);
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                *reinterpret_cast<float4*>(crow + j) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) crow[j] = accum ? crow[j] + f[j] : f[j];
            }
          } else {
            bf16* crow = reinterpret_cast<bf16*>(Cv) + (size_t)row * ldc + col0;
            if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (accum) {
                  const uint4 p = *reinterpret_cast<uint4*>(crow + j);
                  const __nv_bfloat162* ph2 = reinterpret_cast<const __nv_bfloat162*>(&p);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 pf = __bfloat1622float2(ph2[e]);
                    f[j + 2 * e] += pf.x;
                    f[j + 2 * e + 1] += pf.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(f[j], f[j + 1]);
                o.y = pack_bf16x2(f[j + 2], f[j + 3]);
                o.z = pack_bf16x2(f[j + 4], f[j + 5]);
                o.w = pack_bf16x2(f[j + 6], f[j + 7]);
                *reinterpret_cast<uint4*>(crow + j) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) {
                  const float o = accum ? __bfloat162float(crow[j]) + f[j] : f[j];
                  crow[j] = __float2bfloat16(o);
                }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
    }
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
    tmem_dealloc_pair<C::TMEM_COLS>(tmem_base);
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

template <int BN, bool A_MN, bool B_MN>
static int launch(const void* A, const void* B, void* Cp, const void* bias, int M, int N, int K, int lda, int ldb, int ldc, int flags,
                  int* err_word, cudaStream_t stream, int split_k = 1, float* split_ws = nullptr) {
  using C = Cfg<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  else       rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BN / 2, BK);
  else       rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc) return rc;
  static bool attr_set = false;
  auto kern = gemm_pair_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return -10;
    attr_set = true;
  }
  const int num_kb = (K + BK - 1) / BK;
  if (split_k < 1 || split_ws == nullptr) split_k = 1;
  int kb_per = (num_kb + split_k - 1) / split_k;
  split_k = (num_kb + kb_per - 1) / kb_per;            // no empty slices
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN) * split_k;
  int pairs = sm_count() / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<2 * pairs, 192, C::SMEM_BYTES, stream>>>(tmA, tmB, Cp, reinterpret_cast<const bf16*>(bias), M, N, K, ldc, flags, err_word, nullptr, nullptr,
                                                  split_k, kb_per, split_ws);
  if (cudaGetLastError() != cudaSuccess) return -11;
  if (split_k > 1) return vb_splitk_reduce(split_ws, split_k, M, N, Cp, ldc, bias, (flags & OUT_F32) ? 1 : 0, (flags & ACCUM) ? 1 : 0, stream);
  return 0;
}

static int launch_fp8(const void* A, const void* B, void* Cp, const void* bias, const float* a_scale, const float* b_scale, int M, int N,
                      int K, int lda, int ldb, int ldc, int flags, int* err_word, cudaStream_t stream) {
  using C = Cfg<256>;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM, 2 * BK)) return -1;
  if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, 128, 2 * BK)) return -1;
  static bool attr_set = false;
  auto kern = gemm_pair_kernel<256, false, false, true>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return -10;
    attr_set = true;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
  int pairs = sm_count() / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<2 * pairs, 192, C::SMEM_BYTES, stream>>>(tmA, tmB, Cp, reinterpret_cast<const bf16*>(bias), M, N, K, ldc, flags, err_word, a_scale, b_scale,
                                                  1, (K + 2 * BK - 1) / (2 * BK), nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace pair
}  // namespace vb

// fp8 (e4m3) GEMM on SM pairs: C[M,N] = diag(a_scale) (A8 B8^T) diag(b_scale) (+ bias); A8 [M,K], B8 [N,K] row-major bytes,
// lda/ldb in elements (multiples of 16), fp32 accumulation in TMEM, bf16 or fp32 output. a_scale/b_scale may both be null.
extern "C" int vb_gemm_fp8_pair(const void* A, const void* B, void* C, const void* bias, const float* a_scale, const float* b_scale, int M, int N,
                                int K, int lda, int ldb, int ldc, int out_f32, int* err_word, cudaStream_t stream) {
  using namespace vb::pair;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 15) || (ldb & 15)) return -4;
  if ((a_scale == nullptr) != (b_scale == nullptr)) return -2;
  return launch_fp8(A, B, C, bias, a_scale, b_scale, M, N, K, lda, ldb, ldc, out_f32 ? OUT_F32 : 0, err_word, stream);
}

// Same contract as vb_gemm_bf16 without split-K: C[M,N] (+)= op(A) op(B) (+ bias), 256 x 256 tiles on SM pairs.
// Requirements beyond vb_gemm_bf16's: N % 128 == 0 is NOT required (edges are masked), but the K-major B tile is
// loaded in halves of 128 rows, so ldb and the base must satisfy the same 16-byte rules.
// Number of K slices that lets decode-sized problems (few 256 x 256 tiles) occupy the SM pairs: 0 = the paired kernel is no fit.
extern "C" int vb_gemm_pair_plan(int M, int N, int K) {
  using namespace vb::pair;
  if (M <= 128 || (N % 4) != 0) return 0;             // a pair needs rows for both CTAs; the reduce pass works on float4
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  const int pairs = sm_count() / 2;
  if (tiles >= pairs) return 1;
  const int num_kb = (K + BK - 1) / BK;
  int s = pairs / tiles;
  while (s > 1 && num_kb / s < 8) --s;                // keep at least 8 stages of K per slice
  return s > 8 ? 8 : s;
}

extern "C" int vb_gemm_bf16_pair_splitk(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc,
                                        int out_f32, int accumulate, int split_k, float* split_ws, int* err_word, cudaStream_t stream) {
  using namespace vb::pair;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -4;
  const int flags = (out_f32 ? OUT_F32 : 0) | (accumulate ? ACCUM : 0);
  return launch<256, false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream, split_k, split_ws);
}

extern "C" int vb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb, int ldc,
                                 int a_mn, int b_mn, int out_f32, int accumulate, int* err_word, cudaStream_t stream) {
  using namespace vb::pair;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -4;
  const int flags = (out_f32 ? OUT_F32 : 0) | (accumulate ? ACCUM : 0);
  if (!a_mn && !b_mn) return launch<256, false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream);
  if (!a_mn && b_mn) return launch<256, false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream);
  if (a_mn && b_mn) return launch<256, true, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream);
  return launch<256, true, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, err_word, stream);
}
