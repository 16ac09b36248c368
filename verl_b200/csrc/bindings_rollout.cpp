// torch.ops.verl_b200 bindings of the rollout kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "api.h"

void vb_count_launch(int n);

namespace {
using at::Tensor;
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "verl_b200::", what, " failed with code ", rc);
  vb_count_launch(1);
}

// qkv: [T, (Hq+2Hkv)*128] after RoPE; slots int64 [T]; cache layer [num_blocks, 2, Hkv, 64, 128]
void kv_cache_write(const Tensor& qkv, const Tensor& slots, Tensor& cache, int64_t n_q_heads, int64_t n_kv_heads) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.stride(1) == 1, "kv_cache_write: bad qkv");
  TORCH_CHECK(slots.scalar_type() == at::kLong && slots.is_contiguous() && slots.numel() == qkv.size(0), "kv_cache_write: bad slots");
  TORCH_CHECK(cache.is_contiguous() && cache.size(3) == 64 && cache.size(4) == 128 && cache.size(2) == n_kv_heads, "kv_cache_write: bad cache");
  c10::cuda::CUDAGuard guard(qkv.device());
  const at::BFloat16* base = qkv.data_ptr<at::BFloat16>();
  check_rc(vb_kv_cache_write(base + n_q_heads * 128, base + (n_q_heads + n_kv_heads) * 128, qkv.stride(0), slots.data_ptr<long>(),
                             cache.data_ptr(), (int)n_kv_heads, qkv.size(0), cur_stream()),
           "kv_cache_write");
}

// logits [B, V] bf16 or fp32; rng int64 [2] = (seed, step); writes tokens int64 [B], logprobs fp32 [B]
void sample(const Tensor& logits, double temperature, int64_t top_k, double top_p, const Tensor& rng,
            const c10::optional<Tensor>& row_ids, Tensor& out_token, Tensor& out_logprob) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "sample: bad logits");
  const bool bf = logits.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf || logits.scalar_type() == at::kFloat, "sample: logits must be bf16 or fp32");
  TORCH_CHECK(rng.scalar_type() == at::kLong && rng.numel() >= 2, "sample: rng must be int64 [2]");
  TORCH_CHECK(out_token.scalar_type() == at::kLong && out_logprob.scalar_type() == at::kFloat, "sample: bad outputs");
  const int* rid = nullptr;
  if (row_ids.has_value() && row_ids->defined()) {
    TORCH_CHECK(row_ids->scalar_type() == at::kInt, "sample: row_ids must be int32");
    rid = row_ids->data_ptr<int>();
  }
  c10::cuda::CUDAGuard guard(logits.device());
  check_rc(vb_sample(logits.data_ptr(), bf, logits.stride(0), (int)logits.size(0), (int)logits.size(1), (float)temperature,
                     (int)top_k, (float)top_p, rng.data_ptr<long>(), rid, out_token.data_ptr<long>(),
                     out_logprob.data_ptr<float>(), cur_stream()),
           "sample");
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("kv_cache_write(Tensor qkv, Tensor slots, Tensor(a!) cache, int n_q_heads, int n_kv_heads) -> ()", &kv_cache_write);
  m.def("sample(Tensor logits, float temperature, int top_k, float top_p, Tensor rng, Tensor? row_ids, Tensor(a!) out_token, Tensor(b!) out_logprob) -> ()", &sample);
}
