// Rollout-side kernels: KV-cache scatter and token sampling (temperature / top-k / top-p, with log-probs).
// Replace the sampler and cache ops of vLLM used by the reference
// (verl/workers/rollout/vllm_rollout/vllm_async_server.py:690-697, logprobs_mode processed_logprobs).
#include "common.cuh"

namespace vb {

// k/v rows live inside the fused qkv activation: token t, kv head h at kbase + t*ld + h*128.
// cache layer layout [num_blocks, 2, Hkv, 64, 128]; slot = block*64 + offset (negative slot = skip).
__global__ void kv_cache_write_kernel(const bf16* __restrict__ kbase, const bf16* __restrict__ vbase, long ld,
                                      const long* __restrict__ slots, bf16* __restrict__ cache, int n_kv_heads, long T) {
  const long total = T * n_kv_heads * 16;  // 16 vectors of 8 bf16 per head row
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int vec = i & 15;
    const int h = (i >> 4) % n_kv_heads;
    const long t = (i >> 4) / n_kv_heads;
    const long slot = slots[t];
    if (slot < 0) continue;
    const long blk = slot >> 6, off = slot & 63;
    const uint4 kv = *reinterpret_cast<const uint4*>(kbase + t * ld + h * 128 + vec * 8);
    const uint4 vv = *reinterpret_cast<const uint4*>(vbase + t * ld + h * 128 + vec * 8);
    bf16* kd = cache + (((blk * 2 + 0) * n_kv_heads + h) * 64 + off) * 128 + vec * 8;
    bf16* vd = cache + (((blk * 2 + 1) * n_kv_heads + h) * 64 + off) * 128 + vec * 8;
    *reinterpret_cast<uint4*>(kd) = kv;
    *reinterpret_cast<uint4*>(vd) = vv;
  }
}

__device__ __forceinline__ uint32_t hash_u32(uint32_t a, uint32_t b, uint32_t c) {
  // 3-input integer mix (murmur-style finaliser); statistically adequate for Gumbel noise
  uint32_t h = a * 0x9E3779B1u ^ (b + 0x7F4A7C15u) * 0x85EBCA77u ^ (c + 0x165667B1u) * 0xC2B2AE3Du;
  h ^= h >> 16; h *= 0x7FEB352Du; h ^= h >> 15; h *= 0x846CA68Bu; h ^= h >> 16;
  return h;
}

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long i) {
  if constexpr (sizeof(T) == 2) return __bfloat162float(p[i]); else return p[i];
}

struct BlockRed {
  float* sh;  // >= 64 floats
  __device__ float max(float v) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : -INFINITY;
    r = warp_max(r);
    if (threadIdx.x == 0) sh[32] = r;
    __syncthreads();
    r = sh[32];
    __syncthreads();
    return r;
  }
  __device__ float sum(float v) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) sh[32] = r;
    __syncthreads();
    r = sh[32];
    __syncthreads();
    return r;
  }
};

// One CTA per row. rng[0] = seed, rng[1] = step counter (read from device memory so a captured graph can be replayed).
// temperature == 0 selects greedy decoding. Returned log-prob is that of the chosen token under the *processed*
// distribution (after temperature and top-k/top-p renormalisation).
template <typename T>
__global__ void __launch_bounds__(1024) sample_kernel(const T* __restrict__ logits, long ld, int V, float temperature,
                                                      int top_k, float top_p, const long* __restrict__ rng,
                                                      const int* __restrict__ row_ids, long* __restrict__ out_token,
                                                      float* __restrict__ out_logprob) {
  __shared__ float sh[64];
  __shared__ float best_val[32];
  __shared__ int best_idx[32];
  BlockRed red{sh};
  const int row = blockIdx.x;
  const T* x = logits + (long)row * ld;
  const bool greedy = temperature <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temperature;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, ld_logit(x, i) * inv_t);
  m = red.max(m);
  // threshold on scaled logits for top-k / top-p (values below it are dropped); found by bisection
  float thr = -INFINITY;
  if (!greedy && ((top_k > 0 && top_k < V) || top_p < 1.f)) {
    float s_all = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s_all += __expf(ld_logit(x, i) * inv_t - m);
    s_all = red.sum(s_all);
    float lo = m - 40.f, hi = m;   // keep-set {x >= lo} is everything that matters, {x >= hi} is the arg-max only
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f, mass = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = ld_logit(x, i) * inv_t;
        if (v >= mid) { cnt += 1.f; mass += __expf(v - m); }
      }
      cnt = red.sum(cnt);
      mass = red.sum(mass);
      // keep-set {x >= mid} is still large enough for at least one active filter -> the threshold can move up.
      // With both filters active this converges to max(t_k, t_p), i.e. the intersection of the two keep-sets.
      const bool ok_k = (top_k > 0 && top_k < V) && cnt >= (float)top_k;
      const bool ok_p = (top_p < 1.f) && mass >= top_p * s_all;
      const bool too_big = ok_k || ok_p;
      if (too_big) lo = mid; else hi = mid;
    }
    thr = lo;
  }
  const uint32_t seed = (uint32_t)rng[0], step = (uint32_t)rng[1];
  const uint32_t rid = row_ids ? (uint32_t)row_ids[row] : (uint32_t)row;
  float s = 0.f, bv = -INFINITY;
  int bi = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = ld_logit(x, i) * inv_t;
    if (v < thr) continue;
    s += __expf(v - m);
    float key = v;
    if (!greedy) {
      const uint32_t h = hash_u32(seed ^ (rid * 0x632BE5ABu), step, (uint32_t)i);
      const float u = (h >> 8) * (1.0f / 16777216.0f) + (0.5f / 16777216.0f);
      key = v - __logf(-__logf(u));
    }
    if (key > bv) { bv = key; bi = i; }
  }
  s = red.sum(s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { best_val[threadIdx.x >> 5] = bv; best_idx[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    bv = threadIdx.x < (blockDim.x >> 5) ? best_val[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < (blockDim.x >> 5) ? best_idx[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) {
      out_token[row] = bi;
      out_logprob[row] = ld_logit(x, bi) * inv_t - m - __logf(s);
    }
  }
}

}  // namespace vb

using namespace vb;

extern "C" int vb_kv_cache_write(const void* k, const void* v, long ld, const long* slots, void* cache, int n_kv_heads, long T,
                                 cudaStream_t st) {
  if (T == 0) return 0;
  long total = T * n_kv_heads * 16;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  kv_cache_write_kernel<<<grid, 256, 0, st>>>((const bf16*)k, (const bf16*)v, ld, slots, (bf16*)cache, n_kv_heads, T);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int vb_sample(const void* logits, int is_bf16, long ld, int B, int V, float temperature, int top_k, float top_p,
                         const long* rng, const int* row_ids, long* out_token, float* out_logprob, cudaStream_t st) {
  if (B == 0) return 0;
  if (is_bf16)
    sample_kernel<bf16><<<B, 1024, 0, st>>>((const bf16*)logits, ld, V, temperature, top_k, top_p, rng, row_ids, out_token, out_logprob);
  else
    sample_kernel<float><<<B, 1024, 0, st>>>((const float*)logits, ld, V, temperature, top_k, top_p, rng, row_ids, out_token, out_logprob);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
