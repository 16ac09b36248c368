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

// rewards / values / mask [B, R] fp32 -> (advantages, returns); whiten: advantages normalised with their masked mean / unbiased variance
std::tuple<Tensor, Tensor> gae(const Tensor& rewards, const Tensor& values, const Tensor& mask, double gamma, double lam, bool whiten) {
  TORCH_CHECK(rewards.is_cuda() && rewards.dim() == 2, "gae: rewards must be a CUDA [B, R] tensor");
  const int64_t n = rewards.numel();
  check_f32(rewards, n, "rewards"); check_f32(values, n, "values"); check_f32(mask, n, "mask");
  c10::cuda::CUDAGuard guard(rewards.device());
  Tensor adv = at::empty_like(rewards), ret = at::empty_like(rewards);
  Tensor stats = at::zeros({3}, rewards.options());
  check_rc(vb_gae(rewards.data_ptr<float>(), values.data_ptr<float>(), mask.data_ptr<float>(), (int)rewards.size(0), (int)rewards.size(1), (float)gamma,
                  (float)lam, whiten, adv.data_ptr<float>(), ret.data_ptr<float>(), stats.data_ptr<float>(), cur_stream()),
           "gae");
  return {adv, ret};
}

// -> (grad wrt vpreds, stats [3] = weighted loss sum, clipped tokens, masked tokens)
std::tuple<Tensor, Tensor> value_loss(const Tensor& vpreds, const Tensor& values, const Tensor& returns, const Tensor& weight, const Tensor& mask,
                                      double clip) {
  const int64_t n = vpreds.numel();
  check_f32(vpreds, n, "vpreds"); check_f32(values, n, "values"); check_f32(returns, n, "returns"); check_f32(weight, n, "weight"); check_f32(mask, n, "mask");
  c10::cuda::CUDAGuard guard(vpreds.device());
  Tensor grad = at::empty_like(vpreds);
  Tensor stats = at::zeros({3}, vpreds.options());
  check_rc(vb_value_loss(vpreds.data_ptr<float>(), values.data_ptr<float>(), returns.data_ptr<float>(), weight.data_ptr<float>(), mask.data_ptr<float>(), n,
                         (float)clip, grad.data_ptr<float>(), stats.data_ptr<float>(), cur_stream()),
           "value_loss");
  return {grad, stats};
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("gae(Tensor rewards, Tensor values, Tensor mask, float gamma, float lam, bool whiten) -> (Tensor, Tensor)", &gae);
  m.def("value_loss(Tensor vpreds, Tensor values, Tensor returns, Tensor weight, Tensor mask, float clip) -> (Tensor, Tensor)", &value_loss);
  m.def("ppo_loss(Tensor lp, Tensor old_lp, Tensor? ref_lp, Tensor adv, Tensor weight, Tensor mask, Tensor? is_w, float clip_lo, float clip_hi, float clip_c, int kl_type, float kl_coef) -> (Tensor, Tensor, Tensor)", &ppo_loss);
  m.def("grpo_advantage(Tensor scores, Tensor group, int G, Tensor mask, float eps, bool norm_by_std) -> Tensor", &grpo_advantage);
}

at::Tensor& vb_status_tensor(int dev);

namespace {
// y[R, N] = x[R, K] @ w[e]^T per 128-row block (w [E, N, K]); transposed = true reads w [E, K, N] as the dgrad operand.
Tensor gemm_grouped(const Tensor& x, const Tensor& w, const Tensor& blk_expert, bool transposed) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "gemm_grouped: bad x");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 3 && w.is_contiguous(), "gemm_grouped: w must be contiguous [E, N, K]");
  TORCH_CHECK(blk_expert.is_cuda() && blk_expert.scalar_type() == at::kInt && blk_expert.numel() * 128 == x.size(0), "gemm_grouped: bad block table");
  const int R = x.size(0), K = x.size(1), E = w.size(0);
  const int N = transposed ? w.size(2) : w.size(1);
  TORCH_CHECK((transposed ? w.size(1) : w.size(2)) == K, "gemm_grouped: K mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::zeros({R, N}, x.options());
  check_rc(vb_gemm_grouped(x.data_ptr(), w.data_ptr(), y.data_ptr(), blk_expert.data_ptr<int>(), R, N, K, E, (int)x.stride(0), N, transposed,
                           vb_status_tensor(x.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_grouped");
  return y;
}

// dw[E, M, N] (+)= dy[rows_e, M]^T @ x[rows_e, N]; expert_rng int32 [E, 2] = (first block, end block)
void gemm_grouped_wgrad(const Tensor& dy, const Tensor& x, const Tensor& expert_rng, Tensor& dw, bool accumulate) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16 && dy.stride(1) == 1 && x.stride(1) == 1, "gemm_grouped_wgrad: bad operands");
  TORCH_CHECK(expert_rng.is_cuda() && expert_rng.scalar_type() == at::kInt && expert_rng.is_contiguous() && expert_rng.dim() == 2 && expert_rng.size(1) == 2, "gemm_grouped_wgrad: bad ranges");
  TORCH_CHECK(dw.is_contiguous() && dw.dim() == 3 && dw.size(1) == dy.size(1) && dw.size(2) == x.size(1) && dw.size(0) == expert_rng.size(0), "gemm_grouped_wgrad: bad dw");
  const bool f32 = dw.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || dw.scalar_type() == at::kBFloat16, "gemm_grouped_wgrad: dw must be fp32 or bf16");
  c10::cuda::CUDAGuard guard(dy.device());
  check_rc(vb_gemm_grouped_wgrad(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), expert_rng.data_ptr<int>(), (int)dy.size(0), (int)dy.size(1), (int)x.size(1),
                                 (int)dw.size(0), (int)dy.stride(0), (int)x.stride(0), f32, accumulate, vb_status_tensor(dy.get_device()).data_ptr<int>(),
                                 cur_stream()),
           "gemm_grouped_wgrad");
}
// Expert-parallel dispatch fused into the grouped GEMM. src_ptrs: CPU int64 [world] token buffers ([*, K] bf16, row stride ld_src)
// reachable from this GPU; row_src int32 [R]: (rank << 24) | row, or -1 for padding rows; stage [R, K] bf16 receives the gathered
// operand (kept for the backward pass), flags int32 [>= R / 128].
Tensor gemm_grouped_dispatch(const Tensor& src_ptrs, int64_t ld_src, const Tensor& row_src, const Tensor& w, const Tensor& blk_expert, Tensor& stage,
                             Tensor& flags, bool transposed) {
  TORCH_CHECK(src_ptrs.scalar_type() == at::kLong && !src_ptrs.is_cuda(), "gemm_grouped_dispatch: pointer table must be a CPU int64 tensor");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 3 && w.is_contiguous(), "gemm_grouped_dispatch: w must be contiguous [E, N, K]");
  // transposed: w is [E, K, N] (the stored [E, out, in] weight read as the input-gradient operand)
  const int R = row_src.numel(), E = w.size(0), N = transposed ? w.size(2) : w.size(1), K = transposed ? w.size(1) : w.size(2);
  TORCH_CHECK(row_src.is_cuda() && row_src.scalar_type() == at::kInt && row_src.is_contiguous(), "gemm_grouped_dispatch: bad row table");
  TORCH_CHECK(blk_expert.is_cuda() && blk_expert.scalar_type() == at::kInt && blk_expert.numel() * 128 == R, "gemm_grouped_dispatch: bad block table");
  TORCH_CHECK(stage.is_cuda() && stage.scalar_type() == at::kBFloat16 && stage.is_contiguous() && stage.numel() >= (int64_t)R * K, "gemm_grouped_dispatch: stage too small");
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.numel() * 128 >= R, "gemm_grouped_dispatch: flags too small");
  c10::cuda::CUDAGuard guard(w.device());
  Tensor y = at::zeros({R, N}, w.options());
  check_rc(vb_gemm_grouped_dispatch(src_ptrs.data_ptr<long>(), (int)src_ptrs.numel(), (int)ld_src, row_src.data_ptr<int>(), w.data_ptr(), y.data_ptr(),
                                    blk_expert.data_ptr<int>(), R, N, K, E, N, transposed, stage.data_ptr(), flags.data_ptr<int>(),
                                    vb_status_tensor(w.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_grouped_dispatch");
  return y;
}

// Combine fused into the epilogue: row r of (x @ w[e]^T) * row_w[r] is stored as row (row_dst[r] & 0xFFFFFF) of rank (row_dst[r] >> 24)'s
// [*, N] bf16 buffer out_ptrs[rank] (row stride ld_out).
void gemm_grouped_combine(const Tensor& x, const Tensor& w, const Tensor& blk_expert, const Tensor& row_dst, const Tensor& row_w, const Tensor& out_ptrs,
                          int64_t ld_out, bool transposed) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "gemm_grouped_combine: bad x");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 3 && w.is_contiguous() && (transposed ? w.size(1) : w.size(2)) == x.size(1),
              "gemm_grouped_combine: w must be contiguous [E, N, K] ([E, K, N] when transposed)");
  const int R = x.size(0), K = x.size(1), E = w.size(0), N = transposed ? w.size(2) : w.size(1);
  TORCH_CHECK(blk_expert.is_cuda() && blk_expert.scalar_type() == at::kInt && blk_expert.numel() * 128 == R, "gemm_grouped_combine: bad block table");
  TORCH_CHECK(row_dst.is_cuda() && row_dst.scalar_type() == at::kInt && row_dst.numel() == R && row_w.is_cuda() && row_w.scalar_type() == at::kFloat &&
                  row_w.numel() == R, "gemm_grouped_combine: bad row tables");
  TORCH_CHECK(out_ptrs.scalar_type() == at::kLong && !out_ptrs.is_cuda(), "gemm_grouped_combine: pointer table must be a CPU int64 tensor");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(vb_gemm_grouped_combine(x.data_ptr(), w.data_ptr(), blk_expert.data_ptr<int>(), row_dst.data_ptr<int>(), row_w.data_ptr<float>(),
                                   out_ptrs.data_ptr<long>(), (int)out_ptrs.numel(), R, N, K, E, (int)x.stride(0), (int)ld_out, transposed,
                                   vb_status_tensor(x.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_grouped_combine");
}

// Row tables of the expert-parallel grouped GEMMs (csrc/moe_tables.cu). idx_all int32 [W, Tc, k], w_all fp32 [W, Tc, k].
// -> (row_src int32 [R], row_dst int32 [R], row_w fp32 [R], blk_expert int32 [R / 128], expert_rng int32 [e_local, 2])
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> ep_row_tables(const Tensor& idx_all, const Tensor& w_all, int64_t rank, int64_t e_local) {
  TORCH_CHECK(idx_all.is_cuda() && idx_all.scalar_type() == at::kInt && idx_all.is_contiguous() && idx_all.dim() == 3, "ep_row_tables: idx_all must be int32 [W, Tc, k]");
  TORCH_CHECK(w_all.is_cuda() && w_all.scalar_type() == at::kFloat && w_all.is_contiguous() && w_all.numel() == idx_all.numel(), "ep_row_tables: bad w_all");
  TORCH_CHECK(idx_all.size(0) <= 128 && idx_all.size(1) * idx_all.size(2) < (1 << 24), "ep_row_tables: rank / row codes would overflow");
  c10::cuda::CUDAGuard guard(idx_all.device());
  const int64_t n_total = idx_all.numel();
  const int Tc = idx_all.size(1), k = idx_all.size(2), lo = (int)(rank * e_local);
  auto iopt = idx_all.options();
  Tensor counts = at::zeros({e_local}, iopt);
  check_rc(vb_ep_count(idx_all.data_ptr<int>(), n_total, lo, (int)e_local, counts.data_ptr<int>(), cur_stream()), "ep_count");
  Tensor counts_h = counts.cpu();                                    // the one host synchronisation: the counts size the buffers
  int64_t n_blocks = 0;
  for (int64_t e = 0; e < e_local; ++e) n_blocks += (counts_h.data_ptr<int>()[e] + 127) / 128;
  if (n_blocks == 0) n_blocks = 1;
  const int64_t R = n_blocks * 128;
  Tensor row_src = at::empty({R}, iopt), row_dst = at::empty({R}, iopt), blk = at::empty({n_blocks}, iopt), rng = at::empty({e_local, 2}, iopt);
  Tensor row_w = at::empty({R}, w_all.options());
  Tensor scratch = at::empty({2 * e_local}, iopt);
  check_rc(vb_ep_fill(idx_all.data_ptr<int>(), w_all.data_ptr<float>(), n_total, Tc, k, lo, (int)e_local, counts.data_ptr<int>(), (int)n_blocks,
                      scratch.data_ptr<int>(), row_src.data_ptr<int>(), row_dst.data_ptr<int>(), row_w.data_ptr<float>(), blk.data_ptr<int>(),
                      rng.data_ptr<int>(), cur_stream()),
           "ep_fill");
  return {row_src, row_dst, row_w, blk, rng};
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("ep_row_tables(Tensor idx_all, Tensor w_all, int rank, int e_local) -> (Tensor, Tensor, Tensor, Tensor, Tensor)", &ep_row_tables);
  m.def("gemm_grouped_dispatch(Tensor src_ptrs, int ld_src, Tensor row_src, Tensor w, Tensor blk_expert, Tensor(a!) stage, Tensor(b!) flags, bool transposed=False) -> Tensor", &gemm_grouped_dispatch);
  m.def("gemm_grouped_combine(Tensor x, Tensor w, Tensor blk_expert, Tensor row_dst, Tensor row_w, Tensor out_ptrs, int ld_out, bool transposed=False) -> ()", &gemm_grouped_combine);
  m.def("gemm_grouped(Tensor x, Tensor w, Tensor blk_expert, bool transposed) -> Tensor", &gemm_grouped);
  m.def("gemm_grouped_wgrad(Tensor dy, Tensor x, Tensor expert_rng, Tensor(a!) dw, bool accumulate) -> ()", &gemm_grouped_wgrad);
}
