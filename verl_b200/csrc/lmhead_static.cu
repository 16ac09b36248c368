// Allocation-free variant of the fused lm_head -> log-prob / entropy forward: the partial-softmax scratch lives in a
// file-scope device array instead of caller- or allocator-provided memory. See lmhead_static.h for the contract.
#include "lmhead_static.h"

#include <stdio.h>

#include <mutex>

#include "api.h"

namespace {

// One copy per device context that loads this module. Holds, in order: per-tile row maxima, sums, x-weighted sums
// (each ceil(V/256) * M floats) and the label logits (M floats).
static __device__ __align__(256) float g_lmhead_scratch[VB_LMHEAD_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of the scratch for the current device; looked up once per device.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_lmhead_scratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "vb_lmhead_logprob_fwd_static: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" long vb_lmhead_static_capacity_floats(void) { return VB_LMHEAD_STATIC_SCRATCH_FLOATS; }

extern "C" int vb_lmhead_logprob_fwd_static(const void* h, const void* W, const long* labels, int M, int V, int K, int ldh, int ldw,
                                            float inv_temp, float* logp, float* ent, float* lse, int* err_word,
                                            cudaStream_t stream) {
  if (M <= 0) return 0;
  if (V <= 0 || K <= 0) return -3;
  const long need = vb_lmhead_scratch_floats(M, V);
  if (need > VB_LMHEAD_STATIC_SCRATCH_FLOATS) {
    fprintf(stderr,
            "vb_lmhead_logprob_fwd_static: M=%d, V=%d need %ld scratch floats but the built-in scratch holds %ld; "
            "pass fewer rows per call\n",
            M, V, need, (long)VB_LMHEAD_STATIC_SCRATCH_FLOATS);
    return VB_STATIC_ERR_TOO_LARGE;
  }
  float* scratch = scratch_for_current_device();
  if (scratch == nullptr) return VB_STATIC_ERR_SETUP;
  // vb_lmhead_logprob_fwd clears the label-logit section of the scratch on the stream before it launches, so nothing
  // of an earlier call on the shared array is read back.
  return vb_lmhead_logprob_fwd(h, W, labels, M, V, K, ldh, ldw, inv_temp, scratch, logp, ent, lse, err_word, stream);
}
