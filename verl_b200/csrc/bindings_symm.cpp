// torch.ops.verl_b200 bindings of the symmetric-memory layer.
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

int64_t symm_alloc(int64_t nbytes) {
  long p = vb_symm_alloc(nbytes);
  TORCH_CHECK(p != 0, "symm_alloc: cudaMalloc of ", nbytes, " bytes failed");
  return p;
}
void symm_free(int64_t ptr) { vb_symm_free(ptr); }
Tensor ipc_get_handle(int64_t ptr) {
  Tensor h = at::empty({64}, at::TensorOptions().dtype(at::kByte));
  TORCH_CHECK(vb_ipc_get_handle(ptr, h.data_ptr<uint8_t>()) == 0, "cudaIpcGetMemHandle failed");
  return h;
}
int64_t ipc_open_handle(const Tensor& h) {
  TORCH_CHECK(h.scalar_type() == at::kByte && h.numel() == 64 && !h.is_cuda(), "ipc_open_handle: need a CPU uint8[64] tensor");
  long p = vb_ipc_open_handle(h.contiguous().data_ptr<uint8_t>());
  TORCH_CHECK(p != 0, "cudaIpcOpenMemHandle failed");
  return p;
}
void ipc_close(int64_t ptr) { vb_ipc_close(ptr); }

// dst (local tensor) <- nbytes from a device pointer that may be another GPU's memory mapped through CUDA IPC. The copy is
// one DMA transfer (cudaMemcpyAsync, no kernel reads the peer's memory); consumers then work on the local copy.
void peer_memcpy(Tensor& dst, int64_t src_ptr, int64_t nbytes) {
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && (int64_t)(dst.numel() * dst.element_size()) >= nbytes, "peer_memcpy: dst too small or not contiguous");
  c10::cuda::CUDAGuard guard(dst.device());
  cudaError_t e = cudaMemcpyAsync(dst.data_ptr(), reinterpret_cast<const void*>(src_ptr), (size_t)nbytes, cudaMemcpyDeviceToDevice,
                                  at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "peer_memcpy: ", cudaGetErrorString(e));
}

// Non-owning tensor view on raw device memory.
Tensor tensor_from_ptr(int64_t ptr, at::IntArrayRef sizes, at::ScalarType dtype) {
  int dev = at::cuda::current_device();
  return at::from_blob(reinterpret_cast<void*>(ptr), sizes, at::TensorOptions().dtype(dtype).device(at::kCUDA, dev));
}

void symm_barrier(const Tensor& pad_ptrs, int64_t rank, int64_t world, int64_t epoch) {
  TORCH_CHECK(pad_ptrs.scalar_type() == at::kLong && !pad_ptrs.is_cuda() && pad_ptrs.numel() >= world, "symm_barrier: bad pointer table");
  int dev = at::cuda::current_device();
  check_rc(vb_symm_barrier(pad_ptrs.data_ptr<long>(), (int)rank, (int)world, (int)epoch, vb_status_tensor(dev).data_ptr<int>(), cur_stream()),
           "symm_barrier");
}

// Barrier whose epoch lives in device memory: no host state per launch, so it can sit inside a captured CUDA graph.
void symm_barrier_auto(const Tensor& pad_ptrs, int64_t rank, int64_t world) {
  TORCH_CHECK(pad_ptrs.scalar_type() == at::kLong && !pad_ptrs.is_cuda() && pad_ptrs.numel() >= world, "symm_barrier_auto: bad pointer table");
  int dev = at::cuda::current_device();
  check_rc(vb_symm_barrier_auto(pad_ptrs.data_ptr<long>(), (int)rank, (int)world, vb_status_tensor(dev).data_ptr<int>(), cur_stream()),
           "symm_barrier_auto");
}

void symm_reduce_scatter(const Tensor& grad_ptrs, int64_t world, int64_t shard_off, Tensor& out, Tensor& sumsq, double scale) {
  TORCH_CHECK(grad_ptrs.scalar_type() == at::kLong && !grad_ptrs.is_cuda(), "symm_reduce_scatter: bad pointer table");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous() && sumsq.scalar_type() == at::kFloat, "symm_reduce_scatter: bad out");
  c10::cuda::CUDAGuard guard(out.device());
  check_rc(vb_symm_reduce_scatter(grad_ptrs.data_ptr<long>(), (int)world, shard_off, out.numel(), (float)scale, out.data_ptr<float>(),
                                  sumsq.data_ptr<float>(), cur_stream()),
           "symm_reduce_scatter");
}

void symm_adamw_allgather(Tensor& p32, Tensor& m, Tensor& v, const Tensor& g, const Tensor& param_ptrs, int64_t world, int64_t shard_off,
                          double lr, double b1, double b2, double eps, double wd, int64_t step, const Tensor& scalars) {
  TORCH_CHECK(p32.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && g.scalar_type() == at::kFloat,
              "symm_adamw_allgather: fp32 tensors expected");
  TORCH_CHECK(g.numel() == p32.numel() && scalars.numel() >= 2, "symm_adamw_allgather: size mismatch");
  c10::cuda::CUDAGuard guard(p32.device());
  check_rc(vb_symm_adamw_allgather(p32.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(),
                                   param_ptrs.data_ptr<long>(), (int)world, shard_off, p32.numel(), (float)lr, (float)b1, (float)b2,
                                   (float)eps, (float)wd, (int)step, scalars.data_ptr<float>(), cur_stream()),
           "symm_adamw_allgather");
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("symm_alloc(int nbytes) -> int", &symm_alloc);
  m.def("symm_free(int ptr) -> ()", &symm_free);
  m.def("ipc_get_handle(int ptr) -> Tensor", &ipc_get_handle);
  m.def("ipc_open_handle(Tensor h) -> int", &ipc_open_handle);
  m.def("ipc_close(int ptr) -> ()", &ipc_close);
  m.def("peer_memcpy(Tensor(a!) dst, int src_ptr, int nbytes) -> ()", &peer_memcpy);
  m.def("tensor_from_ptr(int ptr, int[] sizes, ScalarType dtype) -> Tensor", &tensor_from_ptr);
  m.def("symm_barrier(Tensor pad_ptrs, int rank, int world, int epoch) -> ()", &symm_barrier);
  m.def("symm_barrier_auto(Tensor pad_ptrs, int rank, int world) -> ()", &symm_barrier_auto);
  m.def("symm_reduce_scatter(Tensor grad_ptrs, int world, int shard_off, Tensor(a!) out, Tensor(b!) sumsq, float scale) -> ()", &symm_reduce_scatter);
  m.def("symm_adamw_allgather(Tensor(a!) p32, Tensor(b!) m, Tensor(c!) v, Tensor g, Tensor param_ptrs, int world, int shard_off, float lr, float b1, float b2, float eps, float wd, int step, Tensor scalars) -> ()", &symm_adamw_allgather);
}

namespace {
// C = gather(A segments) @ B^T : a_ptrs int64 CPU [world] pointers to [seg_rows, K] bf16 segments (row stride K).
// Optional staging (`stage` [rows_total, K] bf16, `flags` int32 [rows_total / 128], `epoch` > every earlier call's): remote
// segments then cross NVLink once instead of once per output tile column.
struct Stage {
  void* ptr = nullptr;
  int* flags = nullptr;
};
static Stage stage_of(const c10::optional<Tensor>& stage, const c10::optional<Tensor>& flags, int64_t need_elems, int64_t need_flags) {
  Stage s;
  if (stage.has_value() && stage->defined()) {
    TORCH_CHECK(flags.has_value() && flags->defined(), "staging needs a flags tensor");
    TORCH_CHECK(stage->is_cuda() && stage->scalar_type() == at::kBFloat16 && stage->is_contiguous() && stage->numel() >= need_elems, "bad stage buffer");
    TORCH_CHECK(flags->is_cuda() && flags->scalar_type() == at::kInt && flags->numel() >= need_flags, "bad stage flags");
    s.ptr = stage->data_ptr();
    s.flags = flags->data_ptr<int>();
  }
  return s;
}

// transposed = true: b is stored [K, N] (the weight of the forward pass used for its activation gradient)
void gemm_allgather_a(const Tensor& a_ptrs, int64_t seg_rows, const Tensor& b, Tensor& out, const c10::optional<Tensor>& bias, int64_t rank,
                      const c10::optional<Tensor>& stage, const c10::optional<Tensor>& flags, int64_t epoch, bool transposed) {
  TORCH_CHECK(a_ptrs.scalar_type() == at::kLong && !a_ptrs.is_cuda(), "gemm_allgather_a: pointer table must be a CPU int64 tensor");
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.dim() == 2 && b.stride(1) == 1, "gemm_allgather_a: bad b");
  const int world = a_ptrs.numel(), K = transposed ? b.size(0) : b.size(1), N = transposed ? b.size(1) : b.size(0), M = seg_rows * world;
  TORCH_CHECK(out.size(0) == M && out.size(1) == N && out.scalar_type() == at::kBFloat16 && out.stride(1) == 1, "gemm_allgather_a: bad out");
  const void* bias_p = (bias.has_value() && bias->defined()) ? bias->data_ptr() : nullptr;
  c10::cuda::CUDAGuard guard(b.device());
  const Stage st = stage_of(stage, flags, (int64_t)M * K, M / 128);
  check_rc(vb_gemm_allgather(0, a_ptrs.data_ptr<long>(), world, (int)seg_rows, K, b.data_ptr(), (int)b.stride(0), out.data_ptr(), bias_p, M, N, K,
                             (int)out.stride(0), (int)rank, st.ptr, st.flags, (int)epoch, transposed ? 1 : 0, vb_status_tensor(b.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_allgather_a");
}

// C = A @ gather(B segments)^T : weight rows sharded over ranks (ZeRO-3 style all-gather fused into the consuming GEMM).
void gemm_allgather_b(const Tensor& a, const Tensor& b_ptrs, int64_t seg_rows, Tensor& out, const c10::optional<Tensor>& bias, int64_t rank,
                      const c10::optional<Tensor>& stage, const c10::optional<Tensor>& flags, int64_t epoch) {
  TORCH_CHECK(b_ptrs.scalar_type() == at::kLong && !b_ptrs.is_cuda(), "gemm_allgather_b: pointer table must be a CPU int64 tensor");
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && a.dim() == 2 && a.stride(1) == 1, "gemm_allgather_b: bad a");
  const int world = b_ptrs.numel(), K = a.size(1), M = a.size(0), N = seg_rows * world;
  TORCH_CHECK(out.size(0) == M && out.size(1) == N && out.scalar_type() == at::kBFloat16 && out.stride(1) == 1, "gemm_allgather_b: bad out");
  const void* bias_p = (bias.has_value() && bias->defined()) ? bias->data_ptr() : nullptr;
  c10::cuda::CUDAGuard guard(a.device());
  const Stage st = stage_of(stage, flags, (int64_t)N * K, N / 128);
  check_rc(vb_gemm_allgather(1, b_ptrs.data_ptr<long>(), world, (int)seg_rows, K, a.data_ptr(), (int)a.stride(0), out.data_ptr(), bias_p, M, N, K,
                             (int)out.stride(0), (int)rank, st.ptr, st.flags, (int)epoch, 0, vb_status_tensor(a.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_allgather_b");
}

void gemm_peer_scatter(const Tensor& a, const Tensor& b, const Tensor& out_ptrs, int64_t rank, int64_t rows_per_owner, int64_t slot_elems, bool transposed) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_peer_scatter: bad operands");
  TORCH_CHECK(out_ptrs.scalar_type() == at::kLong && !out_ptrs.is_cuda(), "gemm_peer_scatter: pointer table must be a CPU int64 tensor");
  const int M = a.size(0), K = a.size(1), N = transposed ? b.size(1) : b.size(0), world = out_ptrs.numel();
  TORCH_CHECK((transposed ? b.size(0) : b.size(1)) == K, "gemm_peer_scatter: inner dimensions differ");
  c10::cuda::CUDAGuard guard(a.device());
  check_rc(vb_gemm_peer_scatter(a.data_ptr(), b.data_ptr(), M, N, K, (int)a.stride(0), (int)b.stride(0), N, out_ptrs.data_ptr<long>(), (int)rank,
                                world, (int)rows_per_owner, slot_elems, transposed ? 1 : 0, vb_status_tensor(a.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_peer_scatter");
}

// Ulysses, sequence → heads: (a [M, K] token shard) @ (b [N, K])^T (+bias); head h of the result goes to rank head_rank[h],
// head slot head_slot[h], rows [row_off, row_off + M) of that rank's [*, ld_out] buffer.
void gemm_head_scatter(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias, const Tensor& out_ptrs, int64_t ld_out,
                       int64_t row_off, int64_t head_dim, const Tensor& head_rank, const Tensor& head_slot, bool transposed) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_head_scatter: bad operands");
  TORCH_CHECK(out_ptrs.scalar_type() == at::kLong && !out_ptrs.is_cuda(), "gemm_head_scatter: pointer table must be a CPU int64 tensor");
  TORCH_CHECK(head_rank.scalar_type() == at::kInt && head_slot.scalar_type() == at::kInt && !head_rank.is_cuda() && !head_slot.is_cuda(), "gemm_head_scatter: head tables must be CPU int32");
  const int M = a.size(0), K = a.size(1), N = transposed ? b.size(1) : b.size(0), world = out_ptrs.numel();
  TORCH_CHECK((transposed ? b.size(0) : b.size(1)) == K, "gemm_head_scatter: inner dimensions differ");
  TORCH_CHECK(head_rank.numel() * head_dim == N && head_slot.numel() == head_rank.numel(), "gemm_head_scatter: head tables do not cover N");
  const void* bias_p = (bias.has_value() && bias->defined()) ? bias->data_ptr() : nullptr;
  c10::cuda::CUDAGuard guard(a.device());
  check_rc(vb_gemm_head_scatter(a.data_ptr(), b.data_ptr(), bias_p, M, N, K, (int)a.stride(0), (int)b.stride(0), (int)ld_out, out_ptrs.data_ptr<long>(),
                                world, (int)row_off, (int)head_dim, head_rank.data_ptr<int>(), head_slot.data_ptr<int>(), transposed ? 1 : 0,
                                vb_status_tensor(a.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_head_scatter");
}

// Ulysses, heads → sequence: out [M, N] = A @ b^T where A's K axis is split over ranks: rank r holds columns
// [r * k_per_rank, ...) as rows [row_off, row_off + M) of its [rows_total, k_per_rank] buffer a_ptrs[r].
void gemm_kseg(const Tensor& a_ptrs, int64_t k_per_rank, int64_t rows_total, int64_t row_off, const Tensor& b, Tensor& out,
               const c10::optional<Tensor>& bias, int64_t rank, const c10::optional<Tensor>& stage, const c10::optional<Tensor>& flags, int64_t epoch,
               bool transposed) {
  TORCH_CHECK(a_ptrs.scalar_type() == at::kLong && !a_ptrs.is_cuda(), "gemm_kseg: pointer table must be a CPU int64 tensor");
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.dim() == 2 && b.stride(1) == 1, "gemm_kseg: bad b");
  const int world = a_ptrs.numel(), N = transposed ? b.size(1) : b.size(0), M = out.size(0);
  TORCH_CHECK((transposed ? b.size(0) : b.size(1)) == world * k_per_rank && out.size(1) == N && out.scalar_type() == at::kBFloat16 && out.stride(1) == 1, "gemm_kseg: bad shapes");
  const void* bias_p = (bias.has_value() && bias->defined()) ? bias->data_ptr() : nullptr;
  c10::cuda::CUDAGuard guard(b.device());
  const int64_t Mp = (M + 127) / 128 * 128;
  const Stage st = stage_of(stage, flags, Mp * world * k_per_rank, (Mp / 128) * world);
  check_rc(vb_gemm_kseg(a_ptrs.data_ptr<long>(), world, (int)k_per_rank, (int)k_per_rank, (int)rows_total, (int)row_off, b.data_ptr(), (int)b.stride(0),
                        out.data_ptr(), bias_p, M, N, (int)out.stride(0), (int)rank, st.ptr, st.flags, (int)epoch, transposed ? 1 : 0,
                        vb_status_tensor(b.get_device()).data_ptr<int>(), cur_stream()),
           "gemm_kseg");
}

// Two-launch all-reduce (see vb_gemm_allreduce_sig): out = sum over ranks of (a_r @ b_r^T) (+ residual)
// phase 0 = both launches (the normal call); 1 = only the GEMM that writes and signals, 2 = only the slot sum. The split lets a
// single-GPU test play several ranks: every rank's GEMM first, then every rank's slot sum, so that no launch waits for a later one.
void gemm_allreduce_sig(const Tensor& a, const Tensor& b, const Tensor& out_ptrs, const Tensor& sig_ptrs, int64_t rank, int64_t half_elems,
                        const Tensor& slots_local, const Tensor& sig_local, const c10::optional<Tensor>& residual, Tensor& out, int64_t bn,
                        int64_t split_k, int64_t max_split, int64_t phase) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_allreduce_sig: bad operands");
  TORCH_CHECK(out_ptrs.scalar_type() == at::kLong && !out_ptrs.is_cuda() && sig_ptrs.scalar_type() == at::kLong && !sig_ptrs.is_cuda() &&
                  out_ptrs.numel() == sig_ptrs.numel(), "gemm_allreduce_sig: pointer tables must be CPU int64 tensors of equal length");
  const int M = a.size(0), K = a.size(1), N = b.size(0), world = out_ptrs.numel();
  const int64_t slot_elems = (int64_t)M * N;
  TORCH_CHECK(slot_elems <= half_elems && slots_local.numel() >= 2 * half_elems && out.size(0) == M && out.size(1) == N &&
                  out.scalar_type() == at::kBFloat16 && out.is_contiguous(), "gemm_allreduce_sig: bad out / slot size");
  const void* res = (residual.has_value() && residual->defined()) ? residual->data_ptr() : nullptr;
  c10::cuda::CUDAGuard guard(a.device());
  int* err = vb_status_tensor(a.get_device()).data_ptr<int>();
  int pbn = 0, ps = 1;
  vb_allreduce_plan(M, N, K, &pbn, &ps);
  if (bn > 0) pbn = (int)bn;
  if (split_k > 0) ps = (int)split_k;
  if (ps > max_split) ps = (int)max_split;
  while (ps > 1 && (int64_t)ps * slot_elems > half_elems) --ps;
  if (phase != 2)
    check_rc(vb_gemm_allreduce_sig(a.data_ptr(), b.data_ptr(), M, N, K, (int)a.stride(0), (int)b.stride(0), out_ptrs.data_ptr<long>(), sig_ptrs.data_ptr<long>(),
                                   (int)rank, world, slot_elems, half_elems, pbn, ps, err, cur_stream()),
             "gemm_allreduce_sig");
  if (phase != 1)
    check_rc(vb_slots_reduce_sig(out_ptrs.data_ptr<long>(), sig_local.data_ptr(), (int)rank, world, ps, slot_elems, half_elems, M, N, res, out.data_ptr(), N, err, cur_stream()),
           "slots_reduce_sig");
}

void slots_reduce(const Tensor& slots, int64_t world, int64_t slot_elems, int64_t rows, int64_t cols, const c10::optional<Tensor>& residual, Tensor& out) {
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "slots_reduce: bf16 tensors expected");
  const void* res = (residual.has_value() && residual->defined()) ? residual->data_ptr() : nullptr;
  c10::cuda::CUDAGuard guard(slots.device());
  check_rc(vb_slots_reduce(slots.data_ptr(), (int)world, slot_elems, rows, (int)cols, (int)cols, res, out.data_ptr(), (int)out.stride(0), cur_stream()),
           "slots_reduce");
}
}  // namespace

TORCH_LIBRARY_FRAGMENT(verl_b200, m) {
  m.def("gemm_allgather_a(Tensor a_ptrs, int seg_rows, Tensor b, Tensor(a!) out, Tensor? bias, int rank=0, Tensor? stage=None, Tensor? flags=None, int epoch=0, bool transposed=False) -> ()", &gemm_allgather_a);
  m.def("gemm_allgather_b(Tensor a, Tensor b_ptrs, int seg_rows, Tensor(a!) out, Tensor? bias, int rank=0, Tensor? stage=None, Tensor? flags=None, int epoch=0) -> ()", &gemm_allgather_b);
  m.def("gemm_peer_scatter(Tensor a, Tensor b, Tensor out_ptrs, int rank, int rows_per_owner, int slot_elems, bool transposed=False) -> ()", &gemm_peer_scatter);
  m.def("gemm_head_scatter(Tensor a, Tensor b, Tensor? bias, Tensor out_ptrs, int ld_out, int row_off, int head_dim, Tensor head_rank, Tensor head_slot, bool transposed=False) -> ()", &gemm_head_scatter);
  m.def("gemm_kseg(Tensor a_ptrs, int k_per_rank, int rows_total, int row_off, Tensor b, Tensor(a!) out, Tensor? bias, int rank=0, Tensor? stage=None, Tensor? flags=None, int epoch=0, bool transposed=False) -> ()", &gemm_kseg);
  m.def("gemm_allreduce_sig(Tensor a, Tensor b, Tensor out_ptrs, Tensor sig_ptrs, int rank, int half_elems, Tensor slots_local, Tensor sig_local, Tensor? residual, Tensor(a!) out, int bn=0, int split_k=0, int max_split=8, int phase=0) -> ()", &gemm_allreduce_sig);
  m.def("slots_reduce(Tensor slots, int world, int slot_elems, int rows, int cols, Tensor? residual, Tensor(a!) out) -> ()", &slots_reduce);
}
