// Fused lm_head -> log-prob / entropy forward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference framework. It exists for library users who drive the kernels
// from plain C/C++ or ctypes rather than through the torch bindings, at a moment when device memory cannot be asked
// for: for example a serving or generation loop whose KV cache was sized to take every free byte of the GPU, where a
// fresh allocation may fail outright or make a caching allocator synchronise the device to hand blocks back. The torch
// binding (`lm_head_logprob_fwd`) obtains its partial-softmax scratch from torch's allocator on every call; this
// variant instead keeps the scratch in a fixed array that is part of the loaded module.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch in floats (16 MiB). A call needs vb_lmhead_scratch_floats(M, V) =
// 3 * ceil(V / 256) * M + M floats; e.g. V = 152064 allows up to M = 2352 rows per call, V = 32000 up to M = 11155.
#define VB_LMHEAD_STATIC_SCRATCH_FLOATS (4l * 1024 * 1024)

// Return codes specific to this entry point (others are those of vb_lmhead_logprob_fwd).
#define VB_STATIC_ERR_TOO_LARGE (-20)  // M, V need more scratch than the built-in array holds; nothing was launched
#define VB_STATIC_ERR_SETUP (-21)      // the per-device set-up (symbol address lookup) failed

// Same computation and argument meaning as vb_lmhead_logprob_fwd, minus the scratch argument:
//   h [M, K] bf16 (row stride ldh), W [V, K] bf16 (row stride ldw), labels int64 [M];
//   outputs fp32 [M]: logp, ent (may be null), lse (may be null). All pointers are device pointers owned by the caller.
//
// Rules of use:
//  * This function and what it calls make no allocation call (no cudaMalloc / cudaFree, no torch allocator). The
//    16 MiB scratch array itself belongs to the library's device module: the CUDA runtime places it on a device when
//    the module is first used there, which at the latest is this entry point's first call on that device, and keeps
//    it until the process exits.
//  * The first call on each device therefore does the set-up: it looks up the device address of the built-in scratch
//    (with that device current) and caches it. Make that first call once at start-up, while memory is still
//    available, and before any stream capture is begun.
//  * Every call on a device uses the same scratch array. Calls issued to one stream are ordered and safe; calls that
//    may overlap in time (different streams, or different host threads on different streams) race on the scratch and
//    give wrong results. Serialise them.
//  * The label-logit section of the scratch is cleared on the stream at the start of each call, so a row whose label
//    lies outside [0, V) yields logp = -lse rather than a stale value from an earlier call.
//  * If vb_lmhead_scratch_floats(M, V) exceeds VB_LMHEAD_STATIC_SCRATCH_FLOATS the call is rejected with
//    VB_STATIC_ERR_TOO_LARGE and a message on stderr; split the rows into several calls.
int vb_lmhead_logprob_fwd_static(const void* h, const void* W, const long* labels, int M, int V, int K, int ldh, int ldw,
                                 float inv_temp, float* logp, float* ent, float* lse, int* err_word, cudaStream_t stream);

// Capacity query for callers that want to size their row chunks: returns VB_LMHEAD_STATIC_SCRATCH_FLOATS.
long vb_lmhead_static_capacity_floats(void);

#ifdef __cplusplus
}
#endif
