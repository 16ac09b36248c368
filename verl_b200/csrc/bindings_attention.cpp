// torch.ops.verl_b200 bindings of the attention kernels.
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

// qkv: [T, (Hq+2Hkv)*128] bf16 fused projection rows; tiles: int32 [n_tiles, 4] on device.
// Returns (out [T, Hq*128] bf16, lse [Hq, T] fp32).
std::tuple<Tensor, Tensor> attn_varlen_fwd(const Tensor& qkv, const Tensor& tiles, int64_t n_q_heads, int64_t n_kv_heads,
                                           double scale) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.stride(1) == 1, "attn: bad qkv");
  TORCH_CHECK(qkv.size(1) == (n_q_heads + 2 * n_kv_heads) * 128, "attn: head_dim must be 128");
  TORCH_CHECK(tiles.is_cuda() && tiles.scalar_type() == at::kInt && tiles.is_contiguous(), "attn: bad tile table");
  const int T = qkv.size(0);
  c10::cuda::CUDAGuard guard(qkv.device());
  Tensor out = at::empty({T, n_q_heads * 128}, qkv.options());
  Tensor lse = at::empty({n_q_heads, T}, qkv.options().dtype(at::kFloat));
  const at::BFloat16* base = qkv.data_ptr<at::BFloat16>();
  check_rc(vb_attn_varlen_fwd(base, base + n_q_heads * 128, base + (n_q_heads + n_kv_heads) * 128, qkv.stride(0), T,
                              (int)n_q_heads, (int)n_kv_heads, tiles.data_ptr(), (int)tiles.size(0), out.data_ptr(),
                              out.stride(0), lse.data_ptr<float>(), T, (float)scale,
                              vb_status_tensor(qkv.get_device()).data_ptr<int>(), cur_stream()),
           "attn_varlen_fwd");
  return {out, lse};
}

// Returns dqkv [T, (Hq+2Hkv)*128] bf16.
// bwd_tiles: int32 [n_tiles, 8] = (kv_tok0, kv_row0, seq_tok0, seq_len, q_tile_begin, 0, 0, 0)
Tensor attn_varlen_bwd(const Tensor& qkv, const Tensor& out, const Tensor& dout, const Tensor& lse, const Tensor& bwd_tiles,
                       int64_t n_q_heads, int64_t n_kv_heads, double scale) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.stride(1) == 1, "attn_bwd: bad qkv");
  TORCH_CHECK(out.is_contiguous() && dout.is_contiguous() && dout.scalar_type() == at::kBFloat16, "attn_bwd: bad out/dout");
  TORCH_CHECK(bwd_tiles.is_cuda() && bwd_tiles.scalar_type() == at::kInt && bwd_tiles.is_contiguous() && bwd_tiles.dim() == 2 && bwd_tiles.size(1) == 8,
              "attn_bwd: the work list must be int32 [n_tiles, 8]");
  const int T = qkv.size(0);
  c10::cuda::CUDAGuard guard(qkv.device());
  Tensor dqkv = at::empty({T, (n_q_heads + 2 * n_kv_heads) * 128}, qkv.options());
  Tensor delta = at::empty({n_q_heads, T}, qkv.options().dtype(at::kFloat));
  Tensor dq_acc = at::empty({T, n_q_heads * 128}, qkv.options().dtype(at::kFloat));
  const at::BFloat16* base = qkv.data_ptr<at::BFloat16>();
  at::BFloat16* dbase = dqkv.data_ptr<at::BFloat16>();
  check_rc(vb_attn_varlen_bwd(base, base + n_q_heads * 128, base + (n_q_heads + n_kv_heads) * 128, qkv.stride(0),
                              dout.data_ptr(), out.data_ptr(), out.stride(0), T, (int)n_q_heads, (int)n_kv_heads,
                              bwd_tiles.data_ptr(), (int)bwd_tiles.size(0), lse.data_ptr<float>(), delta.data_ptr<float>(), T,
                              dq_acc.data_ptr<float>(), dbase, dbase + n_q_heads * 128, dbase + (n_q_heads + n_kv_heads) * 128,
                              dqkv.stride(0), (float)scale, vb_status_tensor(qkv.get_device()).data_ptr<int>(), cur_stream()),
           "attn_varlen_bwd");
  return dqkv;
}

// q: [B, Hq*128]; cache: [num_blocks, 2, Hkv, 64, 128]; block_table int32 [B, max_blocks]; kv_lens int32 [B].
// workspace: fp32 scratch of at least B*Hq*num_splits*130 elements when num_splits > 1.
// impl: 0 = pick (transposed GQA kernel when Hq/Hkv <= 16), 1 = generic 128-row query-tile kernel, 2 = transposed GQA kernel.
void attn_paged_decode(const Tensor& q, const Tensor& cache, const Tensor& block_table, const Tensor& kv_lens, Tensor& out,
                       double scale, int64_t num_splits, int64_t max_kv_len, const c10::optional<Tensor>& workspace, int64_t impl) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.is_contiguous(), "paged: bad q");
  TORCH_CHECK(cache.is_contiguous() && cache.dim() == 5 && cache.size(3) == 64 && cache.size(4) == 128, "paged: bad cache");
  TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.is_contiguous() && kv_lens.scalar_type() == at::kInt, "paged: bad tables");
  const int B = q.size(0);
  const int n_kv = cache.size(2);
  const int n_q = q.size(1) / 128;
  float* po = nullptr;
  float* pml = nullptr;
  if (num_splits > 1) {
    TORCH_CHECK(workspace.has_value() && workspace->scalar_type() == at::kFloat &&
                    workspace->numel() >= (int64_t)B * n_q * num_splits * 130, "paged: workspace too small");
    po = workspace->data_ptr<float>();
    pml = po + (int64_t)B * n_q * num_splits * 128;
  }
  c10::cuda::CUDAGuard guard(q.device());
  const bool gqa = impl == 2 || (impl == 0 && n_q / n_kv <= 16);
  auto fn = gqa ? vb_attn_decode_gqa : vb_attn_paged_decode;
  check_rc(fn(q.data_ptr(), q.stride(0), cache.data_ptr(), cache.size(0), block_table.data_ptr<int>(), (int)block_table.size(1),
              kv_lens.data_ptr<int>(), B, n_q, n_kv, out.data_ptr(), out.stride(0), (float)scale, (int)num_splits, (int)max_kv_len, po,
              pml, vb_status_tensor(q.get_device()).data_ptr<int>(), cur_stream()),
           "attn_paged_decode");
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("attn_varlen_fwd(Tensor qkv, Tensor tiles, int n_q_heads, int n_kv_heads, float scale) -> (Tensor, Tensor)", &attn_varlen_fwd);
  m.def("attn_varlen_bwd(Tensor qkv, Tensor out, Tensor dout, Tensor lse, Tensor bwd_tiles, int n_q_heads, int n_kv_heads, float scale) -> Tensor", &attn_varlen_bwd);
  m.def("attn_paged_decode(Tensor q, Tensor cache, Tensor block_table, Tensor kv_lens, Tensor(a!) out, float scale, int num_splits, int max_kv_len, Tensor? workspace, int impl) -> ()", &attn_paged_decode);
}
