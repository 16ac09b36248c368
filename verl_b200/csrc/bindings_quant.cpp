// torch.ops.verl_b200 bindings of the quantisation casts and the weight-delta kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "api.h"

void vb_count_launch(int n);
at::Tensor& vb_status_tensor(int dev);

namespace {
using at::Tensor;
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "verl_b200::", what, " failed with code ", rc);
  vb_count_launch(1);
}

// x [M, N] bf16 -> (y [M, N] float8_e4m3fn, scale [ceil(M/128), ceil(N/128)] fp32, multiply to dequantise)
std::tuple<Tensor, Tensor> fp8_block_cast(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "fp8_block_cast: bad x");
  const int M = x.size(0), N = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty({M, N}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor s = at::empty({(M + 127) / 128, (N + 127) / 128}, x.options().dtype(at::kFloat));
  check_rc(vb_fp8_block_cast(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), s.data_ptr<float>(), M, N, cur_stream()), "fp8_block_cast");
  return {y, s};
}

// x [M, K] bf16 -> (y [M, K] fp8, scale [M, ceil(K/128)] fp32)
std::tuple<Tensor, Tensor> fp8_act_cast(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "fp8_act_cast: bad x");
  const long M = x.size(0);
  const int K = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty({M, K}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor s = at::empty({M, (K + 127) / 128}, x.options().dtype(at::kFloat));
  check_rc(vb_fp8_act_cast(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), s.data_ptr<float>(), M, K, cur_stream()), "fp8_act_cast");
  return {y, s};
}

// x [M, K] bf16 -> (y [M, K] fp8, scale [M] fp32): one scale per row (per token for activations, per output channel for weights)
std::tuple<Tensor, Tensor> fp8_row_cast(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "fp8_row_cast: bad x");
  const long M = x.size(0);
  const int K = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty({M, K}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor s = at::empty({M}, x.options().dtype(at::kFloat));
  check_rc(vb_fp8_row_cast(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), s.data_ptr<float>(), M, K, cur_stream()), "fp8_row_cast");
  return {y, s};
}

// out[M, N] = diag(a_scale) (a8 b8^T) diag(b_scale) (+ bias): e4m3 operands on the tcgen05 f8f6f4 path (SM pairs, 256 x 256 tiles)
Tensor gemm_fp8(const Tensor& a8, const Tensor& b8, const c10::optional<Tensor>& a_scale, const c10::optional<Tensor>& b_scale,
                const c10::optional<Tensor>& bias, bool out_f32) {
  TORCH_CHECK(a8.is_cuda() && b8.is_cuda() && a8.scalar_type() == at::kFloat8_e4m3fn && b8.scalar_type() == at::kFloat8_e4m3fn, "gemm_fp8: operands must be e4m3 CUDA tensors");
  TORCH_CHECK(a8.dim() == 2 && b8.dim() == 2 && a8.size(1) == b8.size(1) && a8.stride(1) == 1 && b8.stride(1) == 1, "gemm_fp8: shapes");
  const int M = a8.size(0), K = a8.size(1), N = b8.size(0);
  const bool scaled = a_scale.has_value() && a_scale->defined();
  TORCH_CHECK(scaled == (b_scale.has_value() && b_scale->defined()), "gemm_fp8: give both scales or none");
  if (scaled) TORCH_CHECK(a_scale->numel() == M && b_scale->numel() == N && a_scale->scalar_type() == at::kFloat && b_scale->scalar_type() == at::kFloat &&
                              a_scale->is_contiguous() && b_scale->is_contiguous(), "gemm_fp8: scales must be fp32 [M] and [N]");
  c10::cuda::CUDAGuard guard(a8.device());
  Tensor out = at::empty({M, N}, a8.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  const void* bp = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N, "gemm_fp8: bias must be bf16 [N]");
    bp = bias->data_ptr();
  }
  int* err = vb_status_tensor(a8.get_device()).data_ptr<int>();
  check_rc(vb_gemm_fp8_pair(a8.data_ptr(), b8.data_ptr(), out.data_ptr(), bp, scaled ? a_scale->data_ptr<float>() : nullptr,
                            scaled ? b_scale->data_ptr<float>() : nullptr, M, N, K, (int)a8.stride(0), (int)b8.stride(0), N, out_f32 ? 1 : 0, err, cur_stream()),
           "gemm_fp8");
  return out;
}

// Block-scaled e4m3 GEMM: a_scale [M, ceil(K/128)] (1 x 128 groups), b_scale [ceil(N/128), ceil(K/128)] (128 x 128 blocks)
Tensor gemm_fp8_block(const Tensor& a8, const Tensor& a_scale, const Tensor& b8, const Tensor& b_scale, const c10::optional<Tensor>& bias, bool out_f32) {
  TORCH_CHECK(a8.is_cuda() && b8.is_cuda() && a8.scalar_type() == at::kFloat8_e4m3fn && b8.scalar_type() == at::kFloat8_e4m3fn, "gemm_fp8_block: operands must be e4m3 CUDA tensors");
  TORCH_CHECK(a8.dim() == 2 && b8.dim() == 2 && a8.size(1) == b8.size(1) && a8.stride(1) == 1 && b8.stride(1) == 1, "gemm_fp8_block: shapes");
  const int M = a8.size(0), K = a8.size(1), N = b8.size(0);
  const int kb = (K + 127) / 128, nb = (N + 127) / 128;
  TORCH_CHECK(a_scale.scalar_type() == at::kFloat && a_scale.is_contiguous() && a_scale.dim() == 2 && a_scale.size(0) == M && a_scale.size(1) == kb,
              "gemm_fp8_block: a_scale must be fp32 [M, ceil(K/128)]");
  TORCH_CHECK(b_scale.scalar_type() == at::kFloat && b_scale.is_contiguous() && b_scale.dim() == 2 && b_scale.size(0) == nb && b_scale.size(1) == kb,
              "gemm_fp8_block: b_scale must be fp32 [ceil(N/128), ceil(K/128)]");
  c10::cuda::CUDAGuard guard(a8.device());
  Tensor out = at::empty({M, N}, a8.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  const void* bp = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N, "gemm_fp8_block: bias must be bf16 [N]");
    bp = bias->data_ptr();
  }
  int* err = vb_status_tensor(a8.get_device()).data_ptr<int>();
  check_rc(vb_gemm_fp8_block(a8.data_ptr(), b8.data_ptr(), out.data_ptr(), a_scale.data_ptr<float>(), b_scale.data_ptr<float>(), bp, M, N, K,
                             (int)a8.stride(0), (int)b8.stride(0), N, out_f32 ? 1 : 0, err, cur_stream()),
           "gemm_fp8_block");
  return out;
}

// ptrs: CPU int64 [world] peer pointers of the row shards. Returns (fp8 [M_out, N], scales) and, if keep_bf16, also the
// gathered bf16 rows.
std::tuple<Tensor, Tensor, Tensor> reshard_quant(const Tensor& ptrs, int64_t rows_per_rank, int64_t ld_src, int64_t row_begin, int64_t M_out,
                                                 int64_t N, bool quantize, bool keep_bf16, const Tensor& like) {
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong, "reshard_quant: ptrs must be a CPU int64 tensor");
  TORCH_CHECK(like.is_cuda(), "reshard_quant: `like` selects the device");
  c10::cuda::CUDAGuard guard(like.device());
  Tensor y, s, o;
  if (quantize) {
    y = at::empty({M_out, N}, like.options().dtype(at::kFloat8_e4m3fn));
    s = at::empty({(M_out + 127) / 128, (N + 127) / 128}, like.options().dtype(at::kFloat));
  } else {
    y = at::empty({0}, like.options().dtype(at::kFloat8_e4m3fn));
    s = at::empty({0}, like.options().dtype(at::kFloat));
  }
  o = keep_bf16 ? at::empty({M_out, N}, like.options().dtype(at::kBFloat16)) : at::empty({0}, like.options().dtype(at::kBFloat16));
  check_rc(vb_reshard_quant(ptrs.data_ptr<int64_t>() ? reinterpret_cast<const long*>(ptrs.data_ptr<int64_t>()) : nullptr, (int)ptrs.numel(),
                            (int)rows_per_rank, ld_src, (int)row_begin, quantize ? y.data_ptr() : nullptr, N, quantize ? s.data_ptr<float>() : nullptr,
                            keep_bf16 ? o.data_ptr() : nullptr, N, (int)M_out, (int)N, cur_stream()),
           "reshard_quant");
  return {y, s, o};
}

// Gather rows [row_begin, row_begin + out.size(0)) of a row-sharded bf16 matrix straight into `out` (a [rows, N] view with
// unit inner stride, e.g. a slice of a parameter): no allocation, no intermediate copy. ptrs may be offset by a column.
void reshard_into(const Tensor& ptrs, int64_t rows_per_rank, int64_t ld_src, int64_t row_begin, Tensor& out) {
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong, "reshard_into: ptrs must be a CPU int64 tensor");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.stride(1) == 1, "reshard_into: out must be a bf16 [rows, N] view");
  c10::cuda::CUDAGuard guard(out.device());
  check_rc(vb_reshard_quant(reinterpret_cast<const long*>(ptrs.data_ptr<int64_t>()), (int)ptrs.numel(), (int)rows_per_rank, ld_src, (int)row_begin, nullptr, 0,
                            nullptr, out.data_ptr(), out.stride(0), (int)out.size(0), (int)out.size(1), cur_stream()),
           "reshard_into");
}

Tensor fp4_fake_quant(const Tensor& x, const Tensor& global_amax) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.size(-1) % 16 == 0, "fp4_fake_quant: bad x");
  TORCH_CHECK(global_amax.is_cuda() && global_amax.scalar_type() == at::kFloat && global_amax.numel() == 1, "fp4_fake_quant: bad amax");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  check_rc(vb_fp4_fake_quant(x.data_ptr(), y.data_ptr(), x.numel(), global_amax.data_ptr<float>(), cur_stream()), "fp4_fake_quant");
  return y;
}

// cur, snap: flat 16-bit tensors of equal length (multiple of 8). Returns the number of changed elements; the first
// min(count, cap) (position, value) pairs are in pos_out / val_out. The snapshot is refreshed.
int64_t delta_compact16(const Tensor& cur, Tensor& snap, Tensor& pos_out, Tensor& val_out) {
  TORCH_CHECK(cur.is_cuda() && cur.is_contiguous() && snap.is_contiguous() && cur.element_size() == 2 && snap.element_size() == 2 &&
                  cur.numel() == snap.numel(), "delta_compact16: bad inputs");
  TORCH_CHECK(pos_out.scalar_type() == at::kInt && val_out.element_size() == 2 && pos_out.numel() == val_out.numel(), "delta_compact16: bad outputs");
  c10::cuda::CUDAGuard guard(cur.device());
  Tensor counter = at::zeros({1}, cur.options().dtype(at::kLong));
  check_rc(vb_delta_compact16(cur.data_ptr(), snap.data_ptr(), cur.numel(), pos_out.data_ptr<int>(), val_out.data_ptr(),
                              reinterpret_cast<unsigned long long*>(counter.data_ptr<int64_t>()), pos_out.numel(), cur_stream()),
           "delta_compact16");
  return counter.item<int64_t>();
}

void delta_apply16(Tensor& dst, const Tensor& pos, const Tensor& val, int64_t count) {
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.element_size() == 2 && pos.scalar_type() == at::kInt && val.element_size() == 2,
              "delta_apply16: bad inputs");
  TORCH_CHECK(count <= pos.numel() && count <= val.numel(), "delta_apply16: count exceeds the buffers");
  c10::cuda::CUDAGuard guard(dst.device());
  check_rc(vb_delta_apply16(dst.data_ptr(), pos.data_ptr<int>(), val.data_ptr(), count, cur_stream()), "delta_apply16");
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("fp8_block_cast(Tensor x) -> (Tensor, Tensor)", &fp8_block_cast);
  m.def("fp8_act_cast(Tensor x) -> (Tensor, Tensor)", &fp8_act_cast);
  m.def("fp8_row_cast(Tensor x) -> (Tensor, Tensor)", &fp8_row_cast);
  m.def("gemm_fp8_block(Tensor a8, Tensor a_scale, Tensor b8, Tensor b_scale, Tensor? bias, bool out_f32=False) -> Tensor", &gemm_fp8_block);
  m.def("gemm_fp8(Tensor a8, Tensor b8, Tensor? a_scale, Tensor? b_scale, Tensor? bias, bool out_f32=False) -> Tensor", &gemm_fp8);
  m.def("fp4_fake_quant(Tensor x, Tensor global_amax) -> Tensor", &fp4_fake_quant);
  m.def("reshard_into(Tensor ptrs, int rows_per_rank, int ld_src, int row_begin, Tensor(a!) out) -> ()", &reshard_into);
  m.def("reshard_quant(Tensor ptrs, int rows_per_rank, int ld_src, int row_begin, int M_out, int N, bool quantize, bool keep_bf16, Tensor like) -> (Tensor, Tensor, Tensor)", &reshard_quant);
  m.def("delta_compact16(Tensor cur, Tensor(a!) snap, Tensor(b!) pos_out, Tensor(c!) val_out) -> int", &delta_compact16);
  m.def("delta_apply16(Tensor(a!) dst, Tensor pos, Tensor val, int count) -> ()", &delta_apply16);
}
