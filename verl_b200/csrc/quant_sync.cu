// Quantisation casts for low-precision rollout weights and the byte-diff kernels of sparse weight synchronisation.
//
//  * blockwise fp8 (e4m3) cast: one CTA per 128x128 block; scale = max(absmax, 1e-10) / 448 is stored (the value to
//    MULTIPLY by when dequantising), y = clamp(x / scale). Reference: verl/utils/kernel/fp8_kernel.py:53-170.
//  * per-row 1x128 group fp8 cast for activations (dynamic activation scheme of the block-scaled GEMM).
//  * NVFP4 fake quantisation for QAT: 16-element groups, group scale rounded to e4m3 relative to a global scale
//    amax / (6 * 448), values rounded to the E2M1 grid {0, .5, 1, 1.5, 2, 3, 4, 6}, then dequantised.
//    Reference: verl/utils/qat/linear.py:42-185.
//  * delta compaction: compare new 16-bit weights with the snapshot of what the receiver already has, emit
//    (position, value) pairs of the elements whose bits changed and refresh the snapshot, all in one pass; and the
//    receiver-side scatter. Reference (torch ops, 4 passes): verl/checkpoint_engine/delta_sync/sparse_gather.py:41-59.
#include <cuda_fp8.h>

#include "common.cuh"

namespace vb {

__device__ __forceinline__ float block_max_256(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    r = warp_max(r);
    if (threadIdx.x == 0) red[0] = r;
  }
  __syncthreads();
  r = red[0];
  __syncthreads();
  return r;
}

// grid (ceil(N/128), ceil(M/128)), 256 threads: thread t owns 8 consecutive columns (t % 16) of rows (t / 16) + 16 i.
__global__ void __launch_bounds__(256) fp8_block_cast_kernel(const bf16* __restrict__ x, long ldx, __nv_fp8_e4m3* __restrict__ y, long ldy,
                                                             float* __restrict__ scale, int M, int N) {
  __shared__ float red[8];
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 128 + (threadIdx.x & 15) * 8;
  const bool vec = (c0 + 8 <= N) && ((ldx & 7) == 0);
  uint4 regs[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + (threadIdx.x >> 4) + 16 * i;
    regs[i] = make_uint4(0, 0, 0, 0);
    if (r < M) {
      if (vec) {
        regs[i] = *reinterpret_cast<const uint4*>(x + (long)r * ldx + c0);
      } else {
        bf16* e = reinterpret_cast<bf16*>(&regs[i]);
        for (int j = 0; j < 8; ++j) e[j] = (c0 + j < N) ? x[(long)r * ldx + c0 + j] : __float2bfloat16(0.f);
      }
    }
    const bf16* e = reinterpret_cast<const bf16*>(&regs[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(e[j])));
  }
  amax = fmaxf(block_max_256(amax, red), 1e-10f);
  const float s = amax / 448.f, inv = 1.f / s;
  if (threadIdx.x == 0) scale[(long)blockIdx.y * gridDim.x + blockIdx.x] = s;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + (threadIdx.x >> 4) + 16 * i;
    if (r >= M) continue;
    const bf16* e = reinterpret_cast<const bf16*>(&regs[i]);
    __nv_fp8_e4m3 q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = __nv_fp8_e4m3(fminf(fmaxf(__bfloat162float(e[j]) * inv, -448.f), 448.f));
    if (c0 + 8 <= N && (ldy & 7) == 0) {
      *reinterpret_cast<uint2*>(y + (long)r * ldy + c0) = *reinterpret_cast<const uint2*>(q);
    } else {
      for (int j = 0; j < 8 && c0 + j < N; ++j) y[(long)r * ldy + c0 + j] = q[j];
    }
  }
}

// Reshard + requantise: the source matrix is split by rows over `world` ranks (rank r holds rows [r * rows_per_rank, ...)
// of a tensor-parallel or flat shard) and is read straight from the peers' memory (plain P2P loads) while the
// destination is this rank's fp8 copy in rollout layout: rows [row_begin, row_begin + M_out) of the full matrix, block
// scales as in fp8_block_cast_kernel. With out_bf16 != null the gathered rows are also kept in bf16 (no quantisation
// on that copy). One pass over NVLink, no staging buffer.
struct PeerRows {
  const bf16* ptr[16];
};
__global__ void __launch_bounds__(256) reshard_quant_kernel(const __grid_constant__ PeerRows src, int rows_per_rank, long ld_src, int row_begin,
                                                            __nv_fp8_e4m3* __restrict__ y, long ldy, float* __restrict__ scale,
                                                            bf16* __restrict__ out_bf16, long ld_bf16, int M_out, int N) {
  __shared__ float red[8];
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 128 + (threadIdx.x & 15) * 8;
  const bool vec = (c0 + 8 <= N) && ((ld_src & 7) == 0);
  uint4 regs[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + (threadIdx.x >> 4) + 16 * i;
    regs[i] = make_uint4(0, 0, 0, 0);
    if (r < M_out) {
      const int g = row_begin + r;                      // row of the full matrix
      const bf16* base = src.ptr[g / rows_per_rank] + (long)(g % rows_per_rank) * ld_src;
      if (vec) {
        regs[i] = *reinterpret_cast<const uint4*>(base + c0);
      } else {
        bf16* e = reinterpret_cast<bf16*>(&regs[i]);
        for (int j = 0; j < 8; ++j) e[j] = (c0 + j < N) ? base[c0 + j] : __float2bfloat16(0.f);
      }
      if (out_bf16 != nullptr) {
        if (vec && (ld_bf16 & 7) == 0) {
          *reinterpret_cast<uint4*>(out_bf16 + (long)r * ld_bf16 + c0) = regs[i];
        } else {
          const bf16* e = reinterpret_cast<const bf16*>(&regs[i]);
          for (int j = 0; j < 8 && c0 + j < N; ++j) out_bf16[(long)r * ld_bf16 + c0 + j] = e[j];
        }
      }
    }
    const bf16* e = reinterpret_cast<const bf16*>(&regs[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(e[j])));
  }
  if (y == nullptr) return;
  amax = fmaxf(block_max_256(amax, red), 1e-10f);
  const float s = amax / 448.f, inv = 1.f / s;
  if (threadIdx.x == 0) scale[(long)blockIdx.y * gridDim.x + blockIdx.x] = s;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + (threadIdx.x >> 4) + 16 * i;
    if (r >= M_out) continue;
    const bf16* e = reinterpret_cast<const bf16*>(&regs[i]);
    __nv_fp8_e4m3 q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = __nv_fp8_e4m3(fminf(fmaxf(__bfloat162float(e[j]) * inv, -448.f), 448.f));
    if (c0 + 8 <= N && (ldy & 7) == 0) {
      *reinterpret_cast<uint2*>(y + (long)r * ldy + c0) = *reinterpret_cast<const uint2*>(q);
    } else {
      for (int j = 0; j < 8 && c0 + j < N; ++j) y[(long)r * ldy + c0 + j] = q[j];
    }
  }
}

// One warp per (row, 128-column group): scale[row, g] = max(absmax, 1e-10) / 448. K % 8 == 0.
__global__ void __launch_bounds__(256) fp8_act_cast_kernel(const bf16* __restrict__ x, long ldx, __nv_fp8_e4m3* __restrict__ y, long ldy,
                                                           float* __restrict__ scale, long M, int K) {
  const int groups = (K + 127) / 128;
  const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= M * groups) return;
  const long r = w / groups;
  const int g = w % groups, c = g * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (c + 4 <= K) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + c);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(e[j]);
  } else {
    for (int j = 0; j < 4; ++j) v[j] = (c + j < K) ? __bfloat162float(x[r * ldx + c + j]) : 0.f;
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = fmaxf(warp_max(amax), 1e-10f);
  const float s = amax / 448.f, inv = 1.f / s;
  if (lane == 0) scale[r * groups + g] = s;
  __nv_fp8_e4m3 q[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) q[j] = __nv_fp8_e4m3(fminf(fmaxf(v[j] * inv, -448.f), 448.f));
  if (c + 4 <= K) {
    *reinterpret_cast<uint32_t*>(y + r * ldy + c) = *reinterpret_cast<const uint32_t*>(q);
  } else {
    for (int j = 0; j < 4 && c + j < K; ++j) y[r * ldy + c + j] = q[j];
  }
}

__device__ __forceinline__ float e2m1_round(float a) {
  return a <= 0.25f ? 0.f : a < 0.75f ? 0.5f : a <= 1.25f ? 1.f : a < 1.75f ? 1.5f : a <= 2.5f ? 2.f : a < 3.5f ? 3.f : a <= 5.f ? 4.f : 6.f;
}

// One thread per 16-element group (two 16-byte loads). N % 16 == 0.
__global__ void __launch_bounds__(256) fp4_fake_quant_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long n_groups,
                                                             const float* __restrict__ global_amax) {
  const float gs = global_amax[0] / (6.f * 448.f);
  const float gs_safe = gs > 0.f ? gs : 1e-12f;
  for (long g = blockIdx.x * (long)blockDim.x + threadIdx.x; g < n_groups; g += (long)gridDim.x * blockDim.x) {
    uint4 raw[2];
    raw[0] = reinterpret_cast<const uint4*>(x)[2 * g];
    raw[1] = reinterpret_cast<const uint4*>(x)[2 * g + 1];
    const bf16* e = reinterpret_cast<const bf16*>(raw);
    float v[16], amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = __bfloat162float(e[j]);
      amax = fmaxf(amax, fabsf(v[j]));
    }
    float sc = fminf(amax / (6.f * gs_safe), 448.f);
    sc = float(__nv_fp8_e4m3(sc)) * gs;
    if (!(sc >= 1e-5f)) sc = 1.f;
    uint4 out[2];
    bf16* o = reinterpret_cast<bf16*>(out);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float q = e2m1_round(fabsf(v[j]) / sc) * sc;
      o[j] = __float2bfloat16(v[j] >= 0.f ? q : -q);
    }
    reinterpret_cast<uint4*>(y)[2 * g] = out[0];
    reinterpret_cast<uint4*>(y)[2 * g + 1] = out[1];
  }
}

// ---------------------------------------------------------------- byte-diff delta
// 16-bit elements, n % 8 == 0. counter[0] receives the number of changed elements (it may exceed `cap`; pairs beyond
// cap are dropped and the caller falls back to a dense transfer). The snapshot is refreshed in the same pass.
__global__ void __launch_bounds__(256) delta_compact16_kernel(const uint16_t* __restrict__ cur, uint16_t* __restrict__ snap, long n,
                                                              int* __restrict__ pos_out, uint16_t* __restrict__ val_out,
                                                              unsigned long long* __restrict__ counter, long cap) {
  __shared__ unsigned long long base;
  __shared__ int warp_tot[8];
  const long n8 = n >> 3;
  const long iters = (n8 + (long)gridDim.x * blockDim.x - 1) / ((long)gridDim.x * blockDim.x);
  for (long it = 0; it < iters; ++it) {
    const long i = (it * gridDim.x + blockIdx.x) * (long)blockDim.x + threadIdx.x;
    uint4 a = make_uint4(0, 0, 0, 0), b = a;
    if (i < n8) {
      a = reinterpret_cast<const uint4*>(cur)[i];
      b = reinterpret_cast<const uint4*>(snap)[i];
    }
    const uint16_t* ea = reinterpret_cast<const uint16_t*>(&a);
    const uint16_t* eb = reinterpret_cast<const uint16_t*>(&b);
    int cnt = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) cnt += ea[j] != eb[j];
    // exclusive prefix of cnt inside the block
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if ((threadIdx.x & 31) >= o) incl += t;
    }
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = incl;
    __syncthreads();
    int woff = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < (threadIdx.x >> 5)) woff += warp_tot[w];
      total += warp_tot[w];
    }
    if (threadIdx.x == 0) base = total ? atomicAdd(counter, (unsigned long long)total) : 0ull;
    __syncthreads();
    if (cnt) {
      long o = (long)base + woff + incl - cnt;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (ea[j] != eb[j]) {
          if (o < cap) {
            pos_out[o] = (int)(i * 8 + j);
            val_out[o] = ea[j];
          }
          ++o;
        }
      }
      reinterpret_cast<uint4*>(snap)[i] = a;
    }
    __syncthreads();
  }
}

__global__ void delta_apply16_kernel(uint16_t* __restrict__ dst, const int* __restrict__ pos, const uint16_t* __restrict__ val, long count) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < count; i += (long)gridDim.x * blockDim.x) dst[pos[i]] = val[i];
}

// Per-row (per-token / per-output-channel) e4m3 cast: scale[r] = amax(x[r, :]) / 448, y = x / scale. One CTA per row;
// the row is read once into registers (K <= 8 * 256 * 8 elements) or re-read from L2 for longer rows.
__global__ void __launch_bounds__(256) fp8_row_cast_kernel(const bf16* __restrict__ x, long ldx, __nv_fp8_e4m3* __restrict__ y, long ldy,
                                                           float* __restrict__ scale, int K) {
  __shared__ float red[8];
  const long r = blockIdx.x;
  const bf16* xr = x + r * ldx;
  const int nvec = K / 8;
  float amax = 0.f;
  for (int i = threadIdx.x; i < nvec; i += 256) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < K; i += 256) amax = fmaxf(amax, fabsf(__bfloat162float(xr[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float sc = fmaxf(amax, 1e-12f) / 448.f;
  const float inv = 1.f / sc;
  if (threadIdx.x == 0) scale[r] = sc;
  __nv_fp8_e4m3* yr = y + r * ldy;
  for (int i = threadIdx.x; i < nvec; i += 256) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    __nv_fp8_e4m3 o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      o[2 * k] = __nv_fp8_e4m3(f.x * inv);
      o[2 * k + 1] = __nv_fp8_e4m3(f.y * inv);
    }
    reinterpret_cast<uint2*>(yr)[i] = *reinterpret_cast<const uint2*>(o);
  }
  for (int i = nvec * 8 + threadIdx.x; i < K; i += 256) yr[i] = __nv_fp8_e4m3(__bfloat162float(xr[i]) * inv);
}

}  // namespace vb

using namespace vb;

extern "C" {

// x [M, K] bf16 (row stride ldx, 16-byte aligned rows) -> y [M, K] e4m3 (row stride ldy, 8-byte aligned rows), scale [M]
int vb_fp8_row_cast(const void* x, long ldx, void* y, long ldy, float* scale, long M, int K, cudaStream_t st) {
  if (M <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (ldx & 7) || (reinterpret_cast<uintptr_t>(y) & 7) || (ldy & 7)) return -4;
  fp8_row_cast_kernel<<<(unsigned)M, 256, 0, st>>>((const bf16*)x, ldx, (__nv_fp8_e4m3*)y, ldy, scale, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_fp8_block_cast(const void* x, long ldx, void* y, long ldy, float* scale, int M, int N, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  dim3 grid((N + 127) / 128, (M + 127) / 128);
  fp8_block_cast_kernel<<<grid, 256, 0, st>>>((const bf16*)x, ldx, (__nv_fp8_e4m3*)y, ldy, scale, M, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// src_ptrs[r]: rank r's [rows_per_rank, N] bf16 shard (row stride ld_src) as seen from this GPU. Writes rows
// [row_begin, row_begin + M_out) of the full matrix: fp8 + scales into (y, scale) when y != null, bf16 into out_bf16
// when that is != null.
int vb_reshard_quant(const long* src_ptrs, int world, int rows_per_rank, long ld_src, int row_begin, void* y, long ldy, float* scale,
                     void* out_bf16, long ld_bf16, int M_out, int N, cudaStream_t st) {
  if (M_out <= 0 || N <= 0) return 0;
  if (world < 1 || world > 16 || rows_per_rank <= 0 || row_begin < 0 || (long)row_begin + M_out > (long)world * rows_per_rank) return -2;
  PeerRows pr = {};
  for (int r = 0; r < world; ++r) pr.ptr[r] = reinterpret_cast<const bf16*>(src_ptrs[r]);
  dim3 grid((N + 127) / 128, (M_out + 127) / 128);
  reshard_quant_kernel<<<grid, 256, 0, st>>>(pr, rows_per_rank, ld_src, row_begin, (__nv_fp8_e4m3*)y, ldy, scale, (bf16*)out_bf16, ld_bf16,
                                             M_out, N);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_fp8_act_cast(const void* x, long ldx, void* y, long ldy, float* scale, long M, int K, cudaStream_t st) {
  if (M <= 0 || K <= 0) return 0;
  if ((ldx & 3) || (ldy & 3)) return -4;
  const long warps = M * ((K + 127) / 128);
  const long blocks = (warps * 32 + 255) / 256;
  fp8_act_cast_kernel<<<(unsigned)blocks, 256, 0, st>>>((const bf16*)x, ldx, (__nv_fp8_e4m3*)y, ldy, scale, M, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_fp4_fake_quant(const void* x, void* y, long n, const float* global_amax, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n & 15) return -4;
  long blocks = ((n >> 4) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  fp4_fake_quant_kernel<<<(int)blocks, 256, 0, st>>>((const bf16*)x, (bf16*)y, n >> 4, global_amax);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// n must be < 2^31 (positions are int32) and a multiple of 8; counter must be zeroed by the caller.
int vb_delta_compact16(const void* cur, void* snap, long n, int* pos_out, void* val_out, unsigned long long* counter, long cap,
                       cudaStream_t st) {
  if (n <= 0) return 0;
  if ((n & 7) || n >= (1l << 31)) return -4;
  long blocks = ((n >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  delta_compact16_kernel<<<(int)blocks, 256, 0, st>>>((const uint16_t*)cur, (uint16_t*)snap, n, pos_out, (uint16_t*)val_out, counter, cap);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_delta_apply16(void* dst, const int* pos, const void* val, long count, cudaStream_t st) {
  if (count <= 0) return 0;
  long blocks = (count + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  delta_apply16_kernel<<<(int)blocks, 256, 0, st>>>((uint16_t*)dst, pos, (const uint16_t*)val, count);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
