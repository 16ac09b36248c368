// Block-scaled fp8 (e4m3) GEMM for sm_100a: C[M,N] = sum_kb a_scale[m, kb] * b_scale[n / 128, kb] * (A8[m, kb-block] . B8[n, kb-block])
//
// Scale granularity is the DeepSeek-style one used for fp8 rollout weights: 1 x 128 along K for activations
// (a_scale [M, K/128]), 128 x 128 for weights (b_scale [N/128, K/128]). Because the scales change every 128 elements of K
// they cannot be applied once in the epilogue; each K block's product has to be promoted into an fp32 sum with its own
// scale. One pipeline stage therefore holds exactly one K block (128 e4m3 bytes per row = one 128-byte swizzle row):
//
//   warp 0      TMA producer: A[128 x 128 B] and B[128 x 128 B] tiles into a shared-memory ring
//   warp 1      MMA issuer:   4 x tcgen05.mma kind::f8f6f4 (K = 32 each) per stage into one of TWO partial accumulators in
//                             TMEM (128 fp32 columns each), never accumulating across stages
//   warps 2-5   promotion:    wait for a partial, tcgen05.ld its 128 columns, acc[c] += (a_scale * b_scale) * partial[c] in
//                             registers (thread = output row), hand the partial buffer back; after the last K block the row
//                             is cast and stored.
// The promotion of block kb overlaps the MMAs of block kb + 1. Persistent over 128 x 128 output tiles. Every wait is bounded.
// Reference semantics: verl/utils/kernel/fp8_kernel.py (block quantisation) consumed by the fp8 GEMMs of the rollout engine.
#include <cstdlib>

#include "common.cuh"
#include "tma_host.h"

namespace vb {
namespace f8b {

constexpr int BM = 128, BN = 128, BKB = 128;            // BKB: bytes (= e4m3 elements) of K per stage
constexpr int TILE_BYTES = 128 * 128;                   // one operand tile per stage
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int STAGES = 6;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

__global__ void __launch_bounds__(192, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cv,
                      const float* __restrict__ a_scale, const float* __restrict__ b_scale, const bf16* __restrict__ bias, int M, int N,
                      int K, int ldc, int out_f32, int* err_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* pfull_bar = empty_bar + STAGES;   // [2] partial accumulator ready
  uint64_t* pempty_bar = pfull_bar + 2;       // [2] partial accumulator consumed (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
  const int num_kb = (K + BKB - 1) / BKB;
  const int num_tiles = num_m * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&pfull_bar[a], 1);
      mbar_init(&pempty_bar[a], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<256>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, err_word, VB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(sa, &tmA, kb * BKB, m0, &full_bar[s]);
          tma_load_2d(sa + TILE_BYTES, &tmB, kb * BKB, n0, &full_bar[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer: one partial product per K block
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0, false, false);      // e4m3 x e4m3, K-major
      int s = 0;
      uint32_t ph = 0, it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t p = it & 1, pph = (it >> 1) & 1;
          if (!mbar_wait(&pempty_bar[p], pph ^ 1, abort_flag, err_word, VB_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(&full_bar[s], ph, abort_flag, err_word, VB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + TILE_BYTES;
          const uint32_t d_tmem = tmem_base + p * BN;
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k)
            umma_f8(d_tmem, make_sdesc_sw128(sa + k * 32, 16, 1024), make_sdesc_sw128(sb + k * 32, 16, 1024), idesc, k != 0);
          umma_commit(&empty_bar[s]);
          umma_commit(&pfull_bar[p]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ promotion + epilogue (128 threads, thread = row)
    const int q = warp & 3;
    const int nkb_scale = num_kb;                       // scale tensors have K/128 columns
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN;
      const int row = m0 + q * 32 + lane;
      const float* as_row = a_scale + (long)min(row, M - 1) * nkb_scale;
      const float* bs_row = b_scale + (long)(n0 / 128) * nkb_scale;
      float acc[BN];
#pragma unroll
      for (int c = 0; c < BN; ++c) acc[c] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const uint32_t p = it & 1, pph = (it >> 1) & 1;
        const float sc = as_row[kb] * bs_row[kb];
        if (!mbar_wait(&pfull_bar[p], pph, abort_flag, err_word, VB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + p * BN + (uint32_t(q * 32) << 16);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(sc, __uint_as_float(v[j]), acc[c * 32 + j]);
        }
        tc_fence_before();
        mbar_arrive(&pempty_bar[p]);
      }
      if (!ok) break;
      if (row < M) {
#pragma unroll
        for (int c = 0; c < BN; c += 8) {
          const int col = n0 + c;
          if (col >= N) break;
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = acc[c + j] + ((bias != nullptr && col + j < N) ? __bfloat162float(bias[col + j]) : 0.f);
          if (out_f32) {
            float* o = reinterpret_cast<float*>(Cv) + (size_t)row * ldc + col;
            for (int j = 0; j < 8; ++j)
              if (col + j < N) o[j] = f[j];
          } else {
            bf16* o = reinterpret_cast<bf16*>(Cv) + (size_t)row * ldc + col;
            if (col + 8 <= N && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
              uint4 w;
              w.x = pack_bf16x2(f[0], f[1]); w.y = pack_bf16x2(f[2], f[3]);
              w.z = pack_bf16x2(f[4], f[5]); w.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(o) = w;
            } else {
              for (int j = 0; j < 8; ++j)
                if (col + j < N) o[j] = __float2bfloat16(f[j]);
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // a wait was abandoned: give copies and MMAs still in flight time to land before TMEM and the ring go away
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) { __nanosleep(1000); }
    }
    tc_fence_after();
    tmem_dealloc<256>(tmem_base);
  }
}

}  // namespace f8b
}  // namespace vb

// A8 [M, K] and B8 [N, K] e4m3 bytes (row strides lda / ldb in elements, multiples of 16); a_scale [M, ceil(K/128)] and
// b_scale [ceil(N/128), ceil(K/128)] fp32, both contiguous; C bf16 or fp32 with row stride ldc.
extern "C" int vb_gemm_fp8_block(const void* A, const void* B, void* C, const float* a_scale, const float* b_scale, const void* bias, int M,
                                 int N, int K, int lda, int ldb, int ldc, int out_f32, int* err_word, cudaStream_t stream) {
  using namespace vb;
  using namespace vb::f8b;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 15) || (ldb & 15)) return -4;
  if (a_scale == nullptr || b_scale == nullptr) return -2;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM, BKB)) return -1;
  if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, BN, BKB)) return -1;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -10;
    attr_set = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  gemm_fp8_block_kernel<<<grid, 192, SMEM_BYTES, stream>>>(tmA, tmB, C, a_scale, b_scale, reinterpret_cast<const bf16*>(bias), M, N, K, ldc,
                                                           out_f32, err_word);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
