// torch.ops.verl_b200.* bindings: thin argument checks + raw-pointer launches of the extern "C" kernels.
// The kernels themselves do not depend on libtorch.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <atomic>

#include "api.h"

namespace {

using at::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

}  // namespace

// Number of kernel-launching calls made through this library (for benchmark accounting).
static std::atomic<long> g_launch_calls{0};
void vb_count_launch(int n) { g_launch_calls.fetch_add(n, std::memory_order_relaxed); }

// One status word per device, shared by all kernels with bounded waits.
at::Tensor& vb_status_tensor(int dev) {
  using at::Tensor;
  static std::vector<Tensor> words(64);
  if (!words[dev].defined()) {
    words[dev] = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, dev));
  }
  return words[dev];
}

namespace {
using at::Tensor;
Tensor& status_word(int dev) { return vb_status_tensor(dev); }

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "verl_b200::", what, " failed with code ", rc);
  vb_count_launch(1);
}

#define CHECK_CUDA_BF16(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kBFloat16, #t " must be a CUDA bf16 tensor")

// out[M,N] (+)= op(a) op(b) (+ bias). a: [M,K] (a_mn=false) or [K,M] (a_mn=true); b: [N,K] or [K,N].
void gemm(const Tensor& a, const Tensor& b, Tensor& out, const c10::optional<Tensor>& bias, bool a_mn, bool b_mn,
          bool accumulate, int64_t bn) {
  CHECK_CUDA_BF16(a);
  CHECK_CUDA_BF16(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm: 2-D tensors expected");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm: innermost stride must be 1");
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: K mismatch ", K, " vs ", Kb);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm: bad output shape");
  const bool out_f32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(out_f32 || out.scalar_type() == at::kBFloat16, "gemm: out must be bf16 or fp32");
  const void* bias_p = nullptr;
  if (bias.has_value() && bias->defined()) {
    CHECK_CUDA_BF16(*bias);
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "gemm: bad bias");
    bias_p = bias->data_ptr();
  }
  c10::cuda::CUDAGuard guard(a.device());
  int* err = status_word(a.get_device()).data_ptr<int>();
  // Training-sized problems run on SM pairs. Two tile shapes: 256 x 512 (fewer operand bytes per FLOP, TMA-store epilogue;
  // bn == 514 forces it) and 256 x 256 (bn == 512 forces it). bn == 0 takes the wide tile whenever it can keep at least half
  // of the SM pairs busy: measured on the Qwen2.5-7B projections (8192 tokens, all three GEMM roles) it is faster for every
  // shape but N = 3584 forward / input-gradient, where the two are within 4 %.
  const long t512 = ((M + 255) / 256) * ((N + 511) / 512), t256 = ((M + 255) / 256) * ((N + 255) / 256);
  const bool ok512 = vb_gemm_pair512_ok(out.data_ptr(), (int)out.stride(0), out_f32, accumulate) && K >= 256;
  const bool auto512 = ok512 && M >= 256 && N >= 512 && t512 >= 37;
  if ((bn == 514 && ok512) || (bn == 0 && auto512)) {
    check_rc(vb_gemm_bf16_pair512(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_p, (int)M, (int)N, (int)K, (int)a.stride(0),
                                  (int)b.stride(0), (int)out.stride(0), a_mn, b_mn, out_f32, accumulate, err, cur_stream()),
             "gemm_pair512");
    return;
  }
  if (bn == 514) bn = 512;
  const bool pair_fits = t256 >= 74 && K >= 256;
  if (bn == 512 || (bn == 0 && pair_fits)) {
    check_rc(vb_gemm_bf16_pair(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_p, (int)M, (int)N, (int)K, (int)a.stride(0),
                               (int)b.stride(0), (int)out.stride(0), a_mn, b_mn, out_f32, accumulate, err, cur_stream()),
             "gemm_pair");
    return;
  }
  // decode-sized problems (one or two row blocks) with a long K: the paired kernel with K slices reads every B tile once
  // per pair. Measured on B200: M=256,N=3584,K=18944 56.3 us vs 60.5 us for the best single-CTA plan, M=512 76.9 vs 87.0;
  // for K=3584 the single-CTA plans win. bn == 513 forces this path.
  if (!a_mn && !b_mn && (bn == 513 || (bn == 0 && M > 128 && M <= 512 && K >= 8192))) {
    const int s2 = vb_gemm_pair_plan((int)M, (int)N, (int)K);
    if (s2 >= 1) {
      Tensor ws2;
      float* wp = nullptr;
      if (s2 > 1) {
        ws2 = at::empty({(int64_t)s2 * M * N}, a.options().dtype(at::kFloat));
        wp = ws2.data_ptr<float>();
      }
      check_rc(vb_gemm_bf16_pair_splitk(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_p, (int)M, (int)N, (int)K, (int)a.stride(0), (int)b.stride(0),
                                        (int)out.stride(0), out_f32, accumulate, s2, wp, err, cur_stream()),
               "gemm_pair_splitk");
      return;
    }
  }
  int bn_sel = 0, split = 1;
  vb_gemm_plan((int)M, (int)N, (int)K, b_mn, (int)bn == 513 ? 0 : (int)bn, &bn_sel, &split);
  Tensor ws;
  float* ws_p = nullptr;
  if (split > 1) {
    ws = at::empty({(int64_t)split * M * N}, a.options().dtype(at::kFloat));
    ws_p = ws.data_ptr<float>();
  }
  int rc = vb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_p, (int)M, (int)N, (int)K, (int)a.stride(0),
                        (int)b.stride(0), (int)out.stride(0), a_mn, b_mn, out_f32, accumulate, bn_sel, split, ws_p, err,
                        cur_stream());
  check_rc(rc, "gemm");
}

std::tuple<Tensor, Tensor, Tensor> rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& res, const Tensor& w,
                                               double eps, bool write_res) {
  CHECK_CUDA_BF16(x);
  CHECK_CUDA_BF16(w);
  TORCH_CHECK(x.is_contiguous() && x.dim() == 2, "rmsnorm: x must be contiguous [T,H]");
  const int T = x.size(0), H = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  Tensor res_out;
  const void* res_p = nullptr;
  void* res_out_p = nullptr;
  if (res.has_value() && res->defined()) {
    TORCH_CHECK(res->is_contiguous() && res->sizes() == x.sizes(), "rmsnorm: bad residual");
    res_p = res->data_ptr();
    if (write_res) {
      res_out = at::empty_like(x);
      res_out_p = res_out.data_ptr();
    }
  }
  check_rc(vb_rmsnorm_fwd(x.data_ptr(), res_p, w.data_ptr(), y.data_ptr(), res_out_p, rstd.data_ptr<float>(), T, H,
                          (float)eps, cur_stream()),
           "rmsnorm_fwd");
  return {y, res_out.defined() ? res_out : Tensor(), rstd};
}

// returns dx; accumulates into dw (fp32 [H]) when given
Tensor rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                   const c10::optional<Tensor>& dres, c10::optional<Tensor> dw) {
  CHECK_CUDA_BF16(dy);
  CHECK_CUDA_BF16(x);
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous(), "rmsnorm_bwd: contiguous inputs expected");
  const int T = x.size(0), H = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = at::empty_like(x);
  float* dw_p = nullptr;
  if (dw.has_value() && dw->defined()) {
    TORCH_CHECK(dw->scalar_type() == at::kFloat && dw->numel() == H, "rmsnorm_bwd: dw must be fp32 [H]");
    dw_p = dw->data_ptr<float>();
  }
  const void* dres_p = (dres.has_value() && dres->defined()) ? dres->data_ptr() : nullptr;
  check_rc(vb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dres_p, dx.data_ptr(), dw_p,
                          T, H, cur_stream()),
           "rmsnorm_bwd");
  return dx;
}

// in-place rotary embedding on x viewed as [T, nheads, D] with token stride x.stride(0)
void rope_(Tensor& x, const Tensor& pos, const Tensor& cos, const Tensor& sin, int64_t nheads, int64_t D, double sign) {
  CHECK_CUDA_BF16(x);
  TORCH_CHECK(pos.scalar_type() == at::kInt && pos.is_contiguous(), "rope: pos must be int32");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() && sin.is_contiguous(),
              "rope: cos/sin must be contiguous fp32 [max_pos, D/2]");
  TORCH_CHECK(x.stride(-1) == 1 && (x.stride(0) % 8) == 0, "rope: bad strides");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(vb_rope(x.data_ptr(), pos.data_ptr<int>(), cos.data_ptr<float>(), sin.data_ptr<float>(), (int)x.size(0),
                   (int)nheads, (int)D, (long)x.stride(0), (float)sign, cur_stream()),
           "rope");
}

// backward of a row gather with repeated indices: out[u] = sum_j g[order[j]] over j in [offsets[u], offsets[u+1])
Tensor segment_sum_rows(const Tensor& g, const Tensor& order, const Tensor& offsets) {
  CHECK_CUDA_BF16(g);
  TORCH_CHECK(g.is_contiguous() && g.dim() == 2 && g.size(1) % 8 == 0, "segment_sum_rows: contiguous [E, C] with C % 8 == 0 expected");
  TORCH_CHECK(order.is_cuda() && offsets.is_cuda() && order.scalar_type() == at::kLong && offsets.scalar_type() == at::kLong &&
                  order.is_contiguous() && offsets.is_contiguous() && order.numel() == g.size(0) && offsets.numel() >= 1,
              "segment_sum_rows: order [E] / offsets [U + 1] must be contiguous int64 CUDA tensors");
  c10::cuda::CUDAGuard guard(g.device());
  const long U = offsets.numel() - 1;
  Tensor out = at::empty({U, g.size(1)}, g.options());
  check_rc(vb_segment_sum_rows(g.data_ptr(), order.data_ptr<long>(), offsets.data_ptr<long>(), out.data_ptr(), U, (int)g.size(1), cur_stream()),
           "segment_sum_rows");
  return out;
}

Tensor swiglu_fwd(const Tensor& gu) {
  CHECK_CUDA_BF16(gu);
  TORCH_CHECK(gu.is_contiguous() && gu.dim() == 2, "swiglu: contiguous [T,2I] expected");
  const long T = gu.size(0);
  const int I = gu.size(1) / 2;
  c10::cuda::CUDAGuard guard(gu.device());
  Tensor out = at::empty({T, I}, gu.options());
  check_rc(vb_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, I, cur_stream()), "swiglu_fwd");
  return out;
}
Tensor swiglu_bwd(const Tensor& gu, const Tensor& dout) {
  CHECK_CUDA_BF16(gu);
  CHECK_CUDA_BF16(dout);
  TORCH_CHECK(gu.is_contiguous() && dout.is_contiguous(), "swiglu_bwd: contiguous inputs expected");
  const long T = gu.size(0);
  const int I = gu.size(1) / 2;
  c10::cuda::CUDAGuard guard(gu.device());
  Tensor dgu = at::empty_like(gu);
  check_rc(vb_swiglu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), T, I, cur_stream()), "swiglu_bwd");
  return dgu;
}

void adamw_(Tensor& p32, Tensor& m, Tensor& v, const Tensor& g, const c10::optional<Tensor>& p16, double lr, double b1,
            double b2, double eps, double wd, int64_t step, const c10::optional<Tensor>& scalars) {
  TORCH_CHECK(p32.is_cuda() && p32.scalar_type() == at::kFloat && p32.is_contiguous(), "adamw: p32 must be fp32");
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat, "adamw: m, v must be fp32");
  TORCH_CHECK(g.numel() == p32.numel() && g.is_contiguous(), "adamw: grad size mismatch");
  const bool g16 = g.scalar_type() == at::kBFloat16;
  TORCH_CHECK(g16 || g.scalar_type() == at::kFloat, "adamw: grad must be bf16 or fp32");
  void* p16_p = nullptr;
  if (p16.has_value() && p16->defined()) {
    CHECK_CUDA_BF16(*p16);
    TORCH_CHECK(p16->numel() == p32.numel() && p16->is_contiguous(), "adamw: p16 size mismatch");
    p16_p = p16->data_ptr();
  }
  const float* sc = (scalars.has_value() && scalars->defined()) ? scalars->data_ptr<float>() : nullptr;
  c10::cuda::CUDAGuard guard(p32.device());
  check_rc(vb_adamw(p32.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr(), g16, p16_p,
                    p32.numel(), (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, (int)step, sc, cur_stream()),
           "adamw");
}

void sqnorm_(const Tensor& g, Tensor& out) {
  TORCH_CHECK(g.is_cuda() && g.is_contiguous() && out.scalar_type() == at::kFloat, "sqnorm: bad arguments");
  const bool g16 = g.scalar_type() == at::kBFloat16;
  TORCH_CHECK(g16 || g.scalar_type() == at::kFloat, "sqnorm: grad must be bf16 or fp32");
  c10::cuda::CUDAGuard guard(g.device());
  check_rc(vb_sqnorm(g.data_ptr(), g16, g.numel(), out.data_ptr<float>(), cur_stream()), "sqnorm");
}

void clip_coef_(const Tensor& sumsq, double max_norm, Tensor& scalars) {
  TORCH_CHECK(scalars.scalar_type() == at::kFloat && scalars.numel() >= 3, "clip_coef: scalars must be fp32 [>=3]");
  c10::cuda::CUDAGuard guard(sumsq.device());
  check_rc(vb_clip_coef(sumsq.data_ptr<float>(), (float)max_norm, scalars.data_ptr<float>(), cur_stream()), "clip_coef");
}

// Reads (and clears) the device status word; synchronises the current stream.
int64_t take_status() {
  int dev = at::cuda::current_device();
  Tensor& w = status_word(dev);
  int64_t v = w[0].item<int>();
  if (v != 0) w.zero_();
  return v;
}

}  // namespace

TORCH_LIBRARY(verl_b200, m) {
  m.def("gemm(Tensor a, Tensor b, Tensor(a!) out, Tensor? bias, bool a_mn, bool b_mn, bool accumulate, int bn) -> ()", &gemm);
  m.def("rmsnorm_fwd(Tensor x, Tensor? res, Tensor w, float eps, bool write_res) -> (Tensor, Tensor, Tensor)", &rmsnorm_fwd);
  m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd, Tensor? dres, Tensor(a!)? dw) -> Tensor", &rmsnorm_bwd);
  m.def("rope_(Tensor(a!) x, Tensor pos, Tensor cos, Tensor sin, int nheads, int D, float sign) -> ()", &rope_);
  m.def("segment_sum_rows(Tensor g, Tensor order, Tensor offsets) -> Tensor", &segment_sum_rows);
  m.def("swiglu_fwd(Tensor gu) -> Tensor", &swiglu_fwd);
  m.def("swiglu_bwd(Tensor gu, Tensor dout) -> Tensor", &swiglu_bwd);
  m.def("adamw_(Tensor(a!) p32, Tensor(b!) m, Tensor(c!) v, Tensor g, Tensor? p16, float lr, float b1, float b2, float eps, float wd, int step, Tensor? scalars) -> ()", &adamw_);
  m.def("sqnorm_(Tensor g, Tensor(a!) out) -> ()", &sqnorm_);
  m.def("clip_coef_(Tensor sumsq, float max_norm, Tensor(a!) scalars) -> ()", &clip_coef_);
  m.def("take_status() -> int", &take_status);
  m.def("launch_count() -> int", []() -> int64_t { return (int64_t)g_launch_calls.load(); });
}
