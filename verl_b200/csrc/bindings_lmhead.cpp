// torch.ops.verl_b200 bindings of the fused lm_head -> log-prob / entropy kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "api.h"

at::Tensor& vb_status_tensor(int dev);

void vb_count_launch(int n);

namespace {
using at::Tensor;
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "verl_b200::", what, " failed with code ", rc);
  vb_count_launch(1);
}

// Returns (logp [M], entropy [M], lse [M]) in fp32.
std::tuple<Tensor, Tensor, Tensor> lmhead_logprob_fwd(const Tensor& h, const Tensor& w, const Tensor& labels, double inv_temp) {
  TORCH_CHECK(h.is_cuda() && h.scalar_type() == at::kBFloat16 && h.dim() == 2 && h.stride(1) == 1, "lmhead: bad h");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1 && w.size(1) == h.size(1), "lmhead: bad w");
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == h.size(0), "lmhead: bad labels");
  const int M = h.size(0), K = h.size(1), V = w.size(0);
  c10::cuda::CUDAGuard guard(h.device());
  auto fo = h.options().dtype(at::kFloat);
  Tensor logp = at::empty({M}, fo), ent = at::empty({M}, fo), lse = at::empty({M}, fo);
  Tensor scratch = at::empty({vb_lmhead_scratch_floats(M, V)}, fo);
  check_rc(vb_lmhead_logprob_fwd(h.data_ptr(), w.data_ptr(), labels.data_ptr<long>(), M, V, K, (int)h.stride(0), (int)w.stride(0),
                                 (float)inv_temp, scratch.data_ptr<float>(), logp.data_ptr<float>(), ent.data_ptr<float>(),
                                 lse.data_ptr<float>(), vb_status_tensor(h.get_device()).data_ptr<int>(), cur_stream()),
           "lmhead_logprob_fwd");
  return {logp, ent, lse};
}

// dlogits for vocabulary rows [col_offset, col_offset + out.size(1)) of w.
void lmhead_dlogits(const Tensor& h, const Tensor& w_chunk, const Tensor& labels, double inv_temp, int64_t col_offset,
                    const Tensor& lse, const Tensor& ent, const Tensor& g_lp, const c10::optional<Tensor>& g_ent, Tensor& out) {
  const int M = h.size(0), K = h.size(1), Vc = w_chunk.size(0);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == M && out.size(1) == Vc && out.stride(1) == 1, "dlogits: bad out");
  TORCH_CHECK(g_lp.scalar_type() == at::kFloat && g_lp.is_contiguous(), "dlogits: g_lp must be fp32");
  const float* ge = nullptr;
  if (g_ent.has_value() && g_ent->defined()) {
    TORCH_CHECK(g_ent->scalar_type() == at::kFloat && g_ent->is_contiguous(), "dlogits: g_ent must be fp32");
    ge = g_ent->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(h.device());
  check_rc(vb_lmhead_dlogits(h.data_ptr(), w_chunk.data_ptr(), labels.data_ptr<long>(), M, Vc, K, (int)h.stride(0),
                             (int)w_chunk.stride(0), (float)inv_temp, (int)col_offset, lse.data_ptr<float>(), ent.data_ptr<float>(),
                             g_lp.data_ptr<float>(), ge, out.data_ptr(), (int)out.stride(0),
                             vb_status_tensor(h.get_device()).data_ptr<int>(), cur_stream()),
           "lmhead_dlogits");
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("lmhead_logprob_fwd(Tensor h, Tensor w, Tensor labels, float inv_temp) -> (Tensor, Tensor, Tensor)", &lmhead_logprob_fwd);
  m.def("lmhead_dlogits(Tensor h, Tensor w_chunk, Tensor labels, float inv_temp, int col_offset, Tensor lse, Tensor ent, Tensor g_lp, Tensor? g_ent, Tensor(a!) out) -> ()", &lmhead_dlogits);
}
