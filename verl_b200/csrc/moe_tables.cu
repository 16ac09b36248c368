// Row tables of the expert-parallel grouped GEMMs, built on the device.
//
// Input: the routing decisions of ALL ranks' tokens (idx_all [W, Tc, k] expert ids, -1 = no such token; w_all the routing weights).
// Output for the experts [lo, lo + e_local) this rank owns: the (token, slot) pairs routed to them, grouped by expert with every
// expert padded to a multiple of 128 rows:
//   row_src[r] = (source rank << 24) | token             where the gate/up GEMM fetches row r from
//   row_dst[r] = (source rank << 24) | (slot * Tc + token) where the down-projection epilogue stores row r
//   row_w[r]   = routing weight of that pair; padding rows: -1 / -1 / 0
//   blk_expert[b] = local expert of 128-row block b (-1: unused), expert_rng[e] = (first block, end block)
// Three launches (count, offsets, fill) replace some thirty small tensor ops; the only host synchronisation left is reading the
// per-expert counts, which size the buffers. Rows of one expert are placed by an atomic cursor, so their order inside the expert's
// segment varies from run to run; every row is an independent GEMM row, which makes the order irrelevant to the result.
// The reference obtains the equivalent bookkeeping from Megatron-Core's token dispatcher (no counterpart file in its tree).
#include <cuda_runtime.h>

#include <cstdint>

namespace vb {

__global__ void ep_count_kernel(const int* __restrict__ idx_all, long n_total, int lo, int e_local, int* __restrict__ counts) {
  extern __shared__ int hist[];
  for (int i = threadIdx.x; i < e_local; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n_total; i += (long)gridDim.x * blockDim.x) {
    const int e = idx_all[i] - lo;
    if (e >= 0 && e < e_local) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < e_local; i += blockDim.x)
    if (hist[i]) atomicAdd(&counts[i], hist[i]);
}

// one block: padded offsets per expert, block -> expert table, expert block ranges, cursors reset
__global__ void ep_offsets_kernel(const int* __restrict__ counts, int e_local, int n_blocks, int* __restrict__ pad_off, int* __restrict__ cursor,
                                  int* __restrict__ blk_expert, int* __restrict__ expert_rng) {
  __shared__ int total_blocks;
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < e_local; ++e) {
      const int nb = (counts[e] + 127) / 128;
      pad_off[e] = off * 128;
      cursor[e] = 0;
      expert_rng[2 * e] = off;
      expert_rng[2 * e + 1] = off + nb;
      off += nb;
    }
    total_blocks = off;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < n_blocks; b += blockDim.x) {
    int e = -1;
    if (b < total_blocks) {
      for (int x = 0; x < e_local; ++x)                        // a few hundred blocks x at most a few hundred experts: a scan will do
        if (expert_rng[2 * x] <= b && b < expert_rng[2 * x + 1]) { e = x; break; }
    }
    blk_expert[b] = e;
  }
}

__global__ void ep_fill_kernel(const int* __restrict__ idx_all, const float* __restrict__ w_all, long n_total, int Tc, int k, int lo, int e_local,
                               const int* __restrict__ pad_off, int* __restrict__ cursor, int* __restrict__ row_src, int* __restrict__ row_dst,
                               float* __restrict__ row_w) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n_total; i += (long)gridDim.x * blockDim.x) {
    const int e = idx_all[i] - lo;
    if (e < 0 || e >= e_local) continue;
    const int pos = atomicAdd(&cursor[e], 1);
    const int r = pad_off[e] + pos;
    const long tok_flat = i / k;
    const int slot = (int)(i - tok_flat * k);
    const int src = (int)(tok_flat / Tc), token = (int)(tok_flat - (long)src * Tc);
    row_src[r] = (src << 24) | token;
    row_dst[r] = (src << 24) | (slot * Tc + token);
    row_w[r] = w_all[i];
  }
}

}  // namespace vb

using namespace vb;

extern "C" {

// counts[e_local] must be zeroed by the caller.
int vb_ep_count(const int* idx_all, long n_total, int lo, int e_local, int* counts, cudaStream_t st) {
  if (n_total <= 0) return 0;
  if (e_local <= 0 || e_local > 4096) return -2;
  long blocks = (n_total + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  ep_count_kernel<<<(int)blocks, 256, e_local * sizeof(int), st>>>(idx_all, n_total, lo, e_local, counts);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// R = 128 * n_blocks rows; row_src / row_dst are set to -1 and row_w to 0 here before the fill.
// scratch: 2 * e_local ints (padded offsets, cursors).
int vb_ep_fill(const int* idx_all, const float* w_all, long n_total, int Tc, int k, int lo, int e_local, const int* counts, int n_blocks, int* scratch,
               int* row_src, int* row_dst, float* row_w, int* blk_expert, int* expert_rng, cudaStream_t st) {
  if (e_local <= 0 || n_blocks <= 0) return -2;
  const size_t R = (size_t)n_blocks * 128;
  if (cudaMemsetAsync(row_src, 0xFF, R * sizeof(int), st) != cudaSuccess) return -13;
  if (cudaMemsetAsync(row_dst, 0xFF, R * sizeof(int), st) != cudaSuccess) return -13;
  if (cudaMemsetAsync(row_w, 0, R * sizeof(float), st) != cudaSuccess) return -13;
  ep_offsets_kernel<<<1, 256, 0, st>>>(counts, e_local, n_blocks, scratch, scratch + e_local, blk_expert, expert_rng);
  if (n_total > 0) {
    long blocks = (n_total + 255) / 256;
    if (blocks > 148 * 4) blocks = 148 * 4;
    ep_fill_kernel<<<(int)blocks, 256, 0, st>>>(idx_all, w_all, n_total, Tc, k, lo, e_local, scratch, scratch + e_local, row_src, row_dst, row_w);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
