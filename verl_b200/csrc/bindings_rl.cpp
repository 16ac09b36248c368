// torch.ops.verl_b200 bindings of the fused PPO loss and GRPO advantage kernels.
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
const float* fptr(const c10::optional<Tensor>& t) { return (t.has_value() && t->defined()) ? t->data_ptr<float>() : nullptr; }
void check_f32(const Tensor& t, int64_t n, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == n, "ppo_loss: bad ", name);
}

// Returns (loss [1], grad wrt log-probs [same shape], stats [7]); see csrc/rl_kernels.cu for the layout of stats.
std::tuple<Tensor, Tensor, Tensor> ppo_loss(const Tensor& lp, const Tensor& old_lp, const c10::optional<Tensor>& ref_lp, const Tensor& adv,
                                            const Tensor& weight, const Tensor& mask, const c10::optional<Tensor>& is_w, double clip_lo,
                                            double clip_hi, double clip_c, int64_t kl_type, double kl_coef) {
  const int64_t n = lp.numel();
  check_f32(lp, n, "log_probs"); check_f32(old_lp, n, "old_log_probs"); check_f32(adv, n, "advantages");
  check_f32(weight, n, "weight"); check_f32(mask, n, "mask");
  if (ref_lp.has_value() && ref_lp->defined()) check_f32(*ref_lp, n, "ref_log_prob");
  if (is_w.has_value() && is_w->defined()) check_f32(*is_w, n, "rollout_is_weights");
  c10::cuda::CUDAGuard guard(lp.device());
  Tensor grad = at::empty_like(lp);
  Tensor loss = at::zeros({1}, lp.options());
  Tensor stats = at::zeros({7}, lp.options());
  check_rc(vb_ppo_loss(lp.data_ptr<float>(), old_lp.data_ptr<float>(), fptr(ref_lp), adv.data_ptr<float>(), weight.data_ptr<float>(),
                       mask.data_ptr<float>(), fptr(is_w), n, (float)clip_lo, (float)clip_hi, (float)clip_c, (int)kl_type, (float)kl_coef,
                       grad.data_ptr<float>(), loss.data_ptr<float>(), stats.data_ptr<float>(), cur_stream()),
           "ppo_loss");
  return {loss, grad, stats};
}

// scores [B] fp32, group int32 [B] (dense ids < G), mask [B, R] fp32 -> advantages [B, R]
Tensor grpo_advantage(const Tensor& scores, const Tensor& group, int64_t G, const Tensor& mask, double eps, bool norm_by_std) {
  TORCH_CHECK(scores.is_cuda() && scores.scalar_type() == at::kFloat && scores.is_contiguous(), "grpo_advantage: bad scores");
  TORCH_CHECK(group.scalar_type() == at::kInt && group.is_contiguous() && group.numel() == scores.numel(), "grpo_advantage: bad group ids");
  TORCH_CHECK(mask.scalar_type() == at::kFloat && mask.is_contiguous() && mask.dim() == 2 && mask.size(0) == scores.numel(), "grpo_advantage: bad mask");
  c10::cuda::CUDAGuard guard(scores.device());
  Tensor mean = at::empty({G}, scores.options()), stdv = at::empty({G}, scores.options());
  Tensor adv = at::empty_like(mask);
  check_rc(vb_grpo_advantage(scores.data_ptr<float>(), group.data_ptr<int>(), (int)scores.numel(), (int)G, mask.data_ptr<float>(), (int)mask.size(1),
                             (float)eps, norm_by_std, mean.data_ptr<float>(), stdv.data_ptr<float>(), adv.data_ptr<float>(), cur_stream()),
           "grpo_advantage");
  return adv;
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("ppo_loss(Tensor lp, Tensor old_lp, Tensor? ref_lp, Tensor adv, Tensor weight, Tensor mask, Tensor? is_w, float clip_lo, float clip_hi, float clip_c, int kl_type, float kl_coef) -> (Tensor, Tensor, Tensor)", &ppo_loss);
  m.def("grpo_advantage(Tensor scores, Tensor group, int G, Tensor mask, float eps, bool norm_by_std) -> Tensor", &grpo_advantage);
}
