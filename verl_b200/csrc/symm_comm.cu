// Symmetric-memory communication primitives over NVLink peer pointers (one process per GPU, one NVSwitch box).
//
// Buffers are plain cudaMalloc allocations exported with CUDA IPC and mapped by every peer, so a kernel on rank r can
// ld/st rank p's copy directly. On top of that:
//   * device barrier on a signal pad with a bounded spin (gives up after a time limit and records an error status);
//   * gradient reduce-scatter fused with the 1/W scale and the squared-norm partial of the reduced shard;
//   * AdamW on the local fp32 shard fused with the all-gather of the updated bf16 parameters (each thread stores its
//     freshly computed values into every peer's parameter buffer).
// Together they replace FSDP's reduce-scatter / clip / optimizer.step / all-gather sequence of the reference
// (verl/workers/engine/fsdp/transformer_impl.py:792-838, verl/utils/fsdp_utils.py:629-642).
// Only plain peer loads/stores are used (no multicast loads), so the same code runs on any number of GPUs.
#include <string.h>

#include "common.cuh"

namespace vb {

constexpr int MAX_RANKS = 16;

struct PeerTable {
  void* ptr[MAX_RANKS];
};

// ---------------------------------------------------------------- barrier
// flags: per rank an int32[MAX_RANKS] pad inside symmetric memory. Rank r writes `epoch` into peer p's flags[r] and then
// waits until its own flags[p] >= epoch for every p. One block, `world` threads.
__global__ void symm_barrier_kernel(const __grid_constant__ PeerTable pads, int rank, int world, int epoch, int* err_word) {
  const int p = threadIdx.x;
  if (p < world) {
    int* remote = reinterpret_cast<int*>(pads.ptr[p]) + rank;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int* mine = reinterpret_cast<const int*>(pads.ptr[rank]) + p;
    uint64_t t0 = 0;
    uint32_t n = 0;
    while (true) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v >= epoch) break;
      if ((++n & 0xFF) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > VB_WAIT_LIMIT_NS) {
          atomicCAS(err_word, 0, VB_ERR_WAIT_PEER | (p << 8));
          break;
        }
        __nanosleep(200);
      }
    }
  }
}

// Same barrier with the epoch kept in device memory (pad word `AUTO_COUNTER`, flags at `AUTO_FLAGS`), so the launch
// carries no host-side state and can be replayed from a CUDA graph: every replay advances the epoch by one on every rank.
constexpr int AUTO_COUNTER = 256;   // int32 index inside the pad
constexpr int AUTO_FLAGS = 512;
__global__ void symm_barrier_auto_kernel(const __grid_constant__ PeerTable pads, int rank, int world, int* err_word) {
  __shared__ int epoch_s;
  int* my_pad = reinterpret_cast<int*>(pads.ptr[rank]);
  if (threadIdx.x == 0) {
    epoch_s = my_pad[AUTO_COUNTER] + 1;
    my_pad[AUTO_COUNTER] = epoch_s;
  }
  __syncthreads();
  const int epoch = epoch_s;
  const int p = threadIdx.x;
  if (p < world) {
    int* remote = reinterpret_cast<int*>(pads.ptr[p]) + AUTO_FLAGS + rank;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int* mine = my_pad + AUTO_FLAGS + p;
    uint64_t t0 = 0;
    uint32_t n = 0;
    while (true) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v >= epoch) break;
      if ((++n & 0xFF) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > VB_WAIT_LIMIT_NS) {
          atomicCAS(err_word, 0, VB_ERR_WAIT_PEER | (p << 8));
          break;
        }
        __nanosleep(200);
      }
    }
  }
}

// ---------------------------------------------------------------- reduce-scatter (+ scale, + sum of squares)
// out[i] = scale * sum_r grads_r[shard_off + i] for i in [0, n); sumsq += sum out[i]^2. n % 4 == 0.
__global__ void __launch_bounds__(512) symm_reduce_scatter_kernel(const __grid_constant__ PeerTable grads, int world, long shard_off, long n, float scale,
                                                                  float* __restrict__ out, float* __restrict__ sumsq) {
  const long n4 = n >> 2;
  float acc = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int r = 0; r < world; ++r) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.ptr[r]) + shard_off) + i);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  __shared__ float part[32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(sumsq, s);
  }
}

// ---------------------------------------------------------------- AdamW + all-gather
// Updates the local fp32 shard and writes the bf16 result into every rank's parameter buffer at shard_off.
// scalars[0] = gradient scale (clip coefficient), scalars[1] = skip flag. n % 8 == 0.
__global__ void __launch_bounds__(256) symm_adamw_allgather_kernel(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
                                                                   const float* __restrict__ g, const __grid_constant__ PeerTable params, int world,
                                                                   long shard_off, long n, float lr, float b1, float b2, float eps,
                                                                   float wd, float bc1, float bc2, const float* __restrict__ scalars) {
  const float gscale = scalars[0];
  const bool skip = scalars[1] != 0.f;
  const long n8 = n >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float pv[8];
    const float4 p0 = reinterpret_cast<const float4*>(p32)[2 * i], p1 = reinterpret_cast<const float4*>(p32)[2 * i + 1];
    pv[0] = p0.x; pv[1] = p0.y; pv[2] = p0.z; pv[3] = p0.w; pv[4] = p1.x; pv[5] = p1.y; pv[6] = p1.z; pv[7] = p1.w;
    if (!skip) {
      float gv[8], mv[8], vv[8];
      const float4 g0 = reinterpret_cast<const float4*>(g)[2 * i], g1 = reinterpret_cast<const float4*>(g)[2 * i + 1];
      const float4 m0 = reinterpret_cast<const float4*>(m)[2 * i], m1 = reinterpret_cast<const float4*>(m)[2 * i + 1];
      const float4 v0 = reinterpret_cast<const float4*>(v)[2 * i], v1 = reinterpret_cast<const float4*>(v)[2 * i + 1];
      gv[0] = g0.x; gv[1] = g0.y; gv[2] = g0.z; gv[3] = g0.w; gv[4] = g1.x; gv[5] = g1.y; gv[6] = g1.z; gv[7] = g1.w;
      mv[0] = m0.x; mv[1] = m0.y; mv[2] = m0.z; mv[3] = m0.w; mv[4] = m1.x; mv[5] = m1.y; mv[6] = m1.z; mv[7] = m1.w;
      vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gi = gv[j] * gscale;
        mv[j] = b1 * mv[j] + (1.f - b1) * gi;
        vv[j] = b2 * vv[j] + (1.f - b2) * gi * gi;
        pv[j] = pv[j] * (1.f - lr * wd) - (lr / bc1) * (mv[j] / (sqrtf(vv[j]) / bc2 + eps));
      }
      reinterpret_cast<float4*>(p32)[2 * i] = make_float4(pv[0], pv[1], pv[2], pv[3]);
      reinterpret_cast<float4*>(p32)[2 * i + 1] = make_float4(pv[4], pv[5], pv[6], pv[7]);
      reinterpret_cast<float4*>(m)[2 * i] = make_float4(mv[0], mv[1], mv[2], mv[3]);
      reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mv[4], mv[5], mv[6], mv[7]);
      reinterpret_cast<float4*>(v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    }
    uint4 o;
    o.x = pack_bf16x2(pv[0], pv[1]); o.y = pack_bf16x2(pv[2], pv[3]);
    o.z = pack_bf16x2(pv[4], pv[5]); o.w = pack_bf16x2(pv[6], pv[7]);
#pragma unroll 4
    for (int r = 0; r < world; ++r) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(params.ptr[r]) + shard_off) + i;
      *dst = o;
    }
  }
}

}  // namespace vb

using namespace vb;

static PeerTable make_table(const long* ptrs, int world) {
  PeerTable t = {};
  for (int i = 0; i < world && i < MAX_RANKS; ++i) t.ptr[i] = reinterpret_cast<void*>(ptrs[i]);
  return t;
}

extern "C" {

// -------- allocation / IPC plumbing (host)
long vb_symm_alloc(long nbytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, nbytes) != cudaSuccess) return 0;
  cudaMemset(p, 0, nbytes);
  return reinterpret_cast<long>(p);
}
int vb_symm_free(long ptr) { return cudaFree(reinterpret_cast<void*>(ptr)) == cudaSuccess ? 0 : -1; }
int vb_ipc_get_handle(long ptr, unsigned char* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr)) != cudaSuccess) return -1;
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(out64, &h, 64);
  return 0;
}
long vb_ipc_open_handle(const unsigned char* in64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return 0;
  return reinterpret_cast<long>(p);
}
int vb_ipc_close(long ptr) { return cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)) == cudaSuccess ? 0 : -1; }

// -------- kernels
int vb_symm_barrier(const long* pad_ptrs, int rank, int world, int epoch, int* err_word, cudaStream_t st) {
  if (world > MAX_RANKS) return -2;
  symm_barrier_kernel<<<1, 32, 0, st>>>(make_table(pad_ptrs, world), rank, world, epoch, err_word);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_symm_barrier_auto(const long* pad_ptrs, int rank, int world, int* err_word, cudaStream_t st) {
  if (world > MAX_RANKS) return -2;
  symm_barrier_auto_kernel<<<1, 32, 0, st>>>(make_table(pad_ptrs, world), rank, world, err_word);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_symm_reduce_scatter(const long* grad_ptrs, int world, long shard_off, long n, float scale, float* out, float* sumsq,
                           cudaStream_t st) {
  if (world > MAX_RANKS || (n & 3) || (shard_off & 3)) return -2;
  if (n == 0) return 0;
  long blocks = ((n >> 2) + 511) / 512;
  if (blocks > 148 * 4) blocks = 148 * 4;
  symm_reduce_scatter_kernel<<<(int)blocks, 512, 0, st>>>(make_table(grad_ptrs, world), world, shard_off, n, scale, out, sumsq);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int vb_symm_adamw_allgather(float* p32, float* m, float* v, const float* g, const long* param_ptrs, int world, long shard_off,
                            long n, float lr, float b1, float b2, float eps, float wd, int step, const float* scalars,
                            cudaStream_t st) {
  if (world > MAX_RANKS || (n & 7) || (shard_off & 7)) return -2;
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step);
  const float bc2 = sqrtf(1.f - powf(b2, (float)step));
  long blocks = ((n >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  symm_adamw_allgather_kernel<<<(int)blocks, 256, 0, st>>>(p32, m, v, g, make_table(param_ptrs, world), world, shard_off, n, lr, b1, b2,
                                                           eps, wd, bc1, bc2, scalars);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
