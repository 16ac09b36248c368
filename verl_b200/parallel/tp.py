"""Tensor-parallel building blocks whose collectives are fused into the GEMM kernels (NVLink peer memory), with the
NCCL versions kept as baseline/oracle (selected by ``VERL_B200_COMM=nccl``).

* ``AllGatherLinear``   y = all_gather(x_shard) @ W_localᵀ       — column-parallel layer after a sequence-sharded region
  (Megatron sequence parallelism): tiles of x are TMA-loaded straight from the owning rank, nothing is gathered first.
* ``GemmAllReduce``     y = Σ_r x_r @ W_rᵀ  on every rank         — row-parallel layer in the rollout engine: the epilogue
  scatters bf16 partial tiles into every rank's slot buffer, a device barrier and one slot-sum kernel finish it.
* ``GemmReduceScatter`` y_shard = (Σ_r x_r @ W_rᵀ)[rows of rank]   — row-parallel layer feeding a sequence-sharded region.
* ``WeightGatherLinear`` y = x @ all_gather(W_shard)ᵀ              — ZeRO-3 parameter all-gather fused into the consuming GEMM.

The reference reaches these through Megatron-Core/TransformerEngine and vLLM (``verl/workers/engine/megatron/
transformer_impl.py:260-340``, ``verl/workers/rollout/vllm_rollout/vllm_async_server.py:328-418``).
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from verl_b200.ops import _ext
from verl_b200.parallel.symm_mem import SymmetricBuffer

__all__ = ["TPContext", "fused_comm_enabled"]


def fused_comm_enabled() -> bool:
    return os.environ.get("VERL_B200_COMM", "native") == "native" and torch.cuda.is_available() and _ext.available()


class TPContext:
    """Symmetric staging buffers + fused ops for one tensor-parallel group."""

    def __init__(self, group, host_group, max_tokens: int, hidden: int, max_out: int, graph_safe: bool = False,
                 allreduce_mode: str = "signal"):
        self.group, self.host_group = group, host_group
        self.graph_safe = graph_safe      # device-side barrier epochs: the ops may be captured into CUDA graphs
        # "signal": GEMM whose last CTA signals the peers + slot sum that waits for the signals (two launches);
        # "barrier": GEMM with peer-scatter epilogue, device barrier, slot sum, device barrier (the earlier four-launch form)
        self.allreduce_mode = allreduce_mode
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.ops = _ext.ops()
        self.max_tokens, self.hidden, self.max_out = max_tokens, hidden, max_out
        # activations that peers read (sequence-sharded inputs of column-parallel layers)
        self.act = SymmetricBuffer(max_tokens * hidden * 2, group, host_group)
        # slots[src_rank][tokens, out] written by peers' GEMM epilogues
        self.slot_elems = max_tokens * max_out
        self.slots = SymmetricBuffer(self.world * self.slot_elems * 2, group, host_group)
        # signalled all-reduce: double-buffered slots + one signal pad per rank (epoch, CTA counter, per-rank flags)
        # (decode-sized calls slice K; every slice of every rank then owns a slot of tokens x out elements inside one half)
        self.half_elems = self.world * self.slot_elems
        self.slots2 = SymmetricBuffer(2 * self.half_elems * 2, group, host_group)
        self.sig = SymmetricBuffer(256, group, host_group)
        self.sig.tensor(torch.int32, 64).zero_()
        torch.cuda.synchronize()
        self.sig.barrier()
        # local staging of the peers' activation shards (each crosses NVLink once per call) + per-128-row arrival flags
        dev = torch.device("cuda", torch.cuda.current_device())
        self.stage = torch.empty(max_tokens * hidden, dtype=torch.bfloat16, device=dev)
        self.stage_flags = torch.zeros(max(1, max_tokens // 128) + 8, dtype=torch.int32, device=dev)
        self.stage_epoch = 0

    # ------------------------------------------------------------------ all-gather → GEMM
    def stage_activation(self, x_shard: torch.Tensor) -> None:
        """Publish this rank's [T/W, H] shard for the peers (copy into the symmetric buffer, then barrier)."""
        n = x_shard.numel()
        self.act.tensor(torch.bfloat16, n).view_as(x_shard).copy_(x_shard)
        self.act.barrier()

    def allgather_linear(self, x_shard: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                         transposed: bool = False) -> torch.Tensor:
        """``all_gather(x_shard) @ wᵀ`` (``transposed``: ``@ w``, the weight as the forward pass stores it — the activation
        gradient of a row-parallel layer). After the fused call the peers' rows of the gathered operand sit in ``self.stage``."""
        rows = x_shard.shape[0]
        out = torch.empty(rows * self.world, w.shape[1] if transposed else w.shape[0], dtype=torch.bfloat16, device=x_shard.device)
        if fused_comm_enabled() and rows % 128 == 0:
            self.stage_activation(x_shard)
            self.stage_epoch += 1
            self.ops.gemm_allgather_a(self.act.table(), rows, w, out, bias, self.rank, self.stage, self.stage_flags, self.stage_epoch, transposed)
            self.act.barrier()      # nobody overwrites its shard while a peer may still be reading it
            return out
        full = torch.empty(rows * self.world, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        return torch.matmul(full, w) if transposed else torch.nn.functional.linear(full, w, bias)

    def gathered_operand(self, x_shard: torch.Tensor) -> torch.Tensor:
        """The full operand of the last fused ``allgather_linear`` call: the staging buffer holds the peers' rows, this
        rank's own rows (which the kernel read in place) are copied in. Valid until the next fused call."""
        rows, k = x_shard.shape
        full = self.stage[: rows * self.world * k].view(rows * self.world, k)
        full[self.rank * rows:(self.rank + 1) * rows].copy_(x_shard)
        return full

    # ------------------------------------------------------------------ GEMM → all-reduce / reduce-scatter
    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, N = x.shape[0], w.shape[0]
        if fused_comm_enabled() and N % 32 == 0 and T * N <= self.slot_elems and self.allreduce_mode == "signal":
            # two launches: GEMM whose last CTA signals the peers, then a slot sum that waits for their signals
            out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
            self.ops.gemm_allreduce_sig(x, w, self.slots2.table(), self.sig.table(), self.rank, self.half_elems,
                                        self.slots2.tensor(torch.bfloat16), self.sig.tensor(torch.int32, 64), residual, out,
                                        0, 0)
            return out
        if fused_comm_enabled() and N % 32 == 0 and T * N <= self.slot_elems:
            out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
            bar = self.slots.barrier_auto if self.graph_safe else self.slots.barrier
            self.ops.gemm_peer_scatter(x, w, self.slots.table(), self.rank, 0, self.slot_elems)
            bar()
            self.ops.slots_reduce(self.slots.tensor(torch.bfloat16), self.world, self.slot_elems, T, N, residual, out)
            bar()                   # slots may be overwritten by the next call only after everyone has summed them
            return out
        y = torch.nn.functional.linear(x, w)
        dist.all_reduce(y, group=self.group)
        return y + residual if residual is not None else y

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, transposed: bool = False) -> torch.Tensor:
        """``reduce_scatter(x @ wᵀ)`` over rows (``transposed``: ``x @ w`` — the activation gradient of a column-parallel layer)."""
        T, N = x.shape[0], (w.shape[1] if transposed else w.shape[0])
        assert T % self.world == 0
        rows = T // self.world
        if fused_comm_enabled() and N % 32 == 0 and rows * N <= self.slot_elems:
            out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
            self.ops.gemm_peer_scatter(x, w, self.slots.table(), self.rank, rows, self.slot_elems, transposed)
            self.slots.barrier()
            self.ops.slots_reduce(self.slots.tensor(torch.bfloat16), self.world, self.slot_elems, rows, N, None, out)
            self.slots.barrier()
            return out
        y = torch.matmul(x, w) if transposed else torch.nn.functional.linear(x, w)
        out = torch.empty(rows, N, dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y, group=self.group)
        return out

    # ------------------------------------------------------------------ ZeRO-3 weight gather → GEMM
    @staticmethod
    def weight_gather_linear(x: torch.Tensor, w_symm: SymmetricBuffer, shard_rows: int, in_features: int, byte_offset: int = 0,
                             stage: Optional[torch.Tensor] = None, flags: Optional[torch.Tensor] = None, epoch: int = 0) -> torch.Tensor:
        """y = x @ concat_r(W_r)ᵀ with W_r = rank r's [shard_rows, in_features] slice living in ``w_symm``. With ``stage``
        ([rows_total, in_features] bf16) and ``flags`` the remote slices are copied into local memory once by the kernel."""
        ops = _ext.ops()
        out = torch.empty(x.shape[0], shard_rows * w_symm.world, dtype=torch.bfloat16, device=x.device)
        ops.gemm_allgather_b(x, w_symm.table(byte_offset), shard_rows, out, None, w_symm.rank, stage, flags, epoch)
        return out


# ---------------------------------------------------------------------------------------------------------------------
# Autograd glue of Megatron-style tensor parallelism ("f" and "g" of the Megatron-LM paper) and the vocabulary-parallel
# embedding. The reference gets these from Megatron-Core (verl/workers/engine/megatron/transformer_impl.py:260-340).
class _CopyToTP(torch.autograd.Function):
    """Identity in forward; all-reduce of the gradient in backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce in forward; identity in backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_tp(x: torch.Tensor, group) -> torch.Tensor:
    return x if group is None or dist.get_world_size(group) == 1 else _CopyToTP.apply(x, group)


def reduce_from_tp(x: torch.Tensor, group) -> torch.Tensor:
    return x if group is None or dist.get_world_size(group) == 1 else _ReduceFromTP.apply(x, group)


def vocab_parallel_embedding(ids: torch.Tensor, w_local: torch.Tensor, vocab_offset: int, group) -> torch.Tensor:
    """Rows [vocab_offset, vocab_offset + w_local.shape[0]) live on this rank; others contribute zeros, then all-reduce."""
    from verl_b200 import ops

    local = ids - vocab_offset
    mine = (local >= 0) & (local < w_local.shape[0])
    h = ops.embedding(torch.where(mine, local, torch.zeros_like(local)), w_local)
    h = h * mine.unsqueeze(-1).to(h.dtype)
    return reduce_from_tp(h, group)


# ---------------------------------------------------------------------------------------------------------------------
# Megatron-style SEQUENCE parallelism: between the tensor-parallel regions the hidden stream is split over the token axis
# ([T/tp, H] per rank), so norms, residual adds and the pipeline sends work on 1/tp of the tokens. A column-parallel
# layer is entered through an all-gather and a row-parallel layer is left through a reduce-scatter; both are fused into
# the GEMM kernels in forward when a ``TPContext`` is attached (``allgather_linear`` / ``gemm_reduce_scatter``), and run
# as collective + GEMM in backward.
def _all_gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    W = dist.get_world_size(group)
    out = torch.empty(W * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    W = dist.get_world_size(group)
    x = x.contiguous()
    if dist.get_backend(group) == "gloo":          # gloo has no reduce-scatter: all-reduce and keep the own slice
        dist.all_reduce(x, group=group)
        n = x.shape[0] // W
        r = dist.get_rank(group)
        return x[r * n:(r + 1) * n].clone()
    out = torch.empty(x.shape[0] // W, *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


class _GatherFromSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_rows(g, ctx.group), None


class _ReduceScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_rows(g, ctx.group), None


class _GatherFromSPReplicatedGrad(torch.autograd.Function):
    """All-gather whose consumer computes the SAME gradient on every rank (e.g. the hidden states entering a replicated
    loss): backward keeps this rank's slice instead of summing the copies."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.n = group, x.shape[0]
        return _all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        r = dist.get_rank(ctx.group)
        return g[r * ctx.n:(r + 1) * ctx.n].contiguous(), None


def gather_from_sp(x, group, replicated_grad: bool = False):
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _GatherFromSPReplicatedGrad.apply(x, group) if replicated_grad else _GatherFromSP.apply(x, group)


def reduce_scatter_to_sp(x, group):
    return x if group is None or dist.get_world_size(group) == 1 else _ReduceScatterToSP.apply(x, group)


def _dgrad(dy, w):
    """dx = dy @ w (w stored [out, in]) on the tcgen05 GEMM when available."""
    from verl_b200.ops.functional import gemm, use_native

    return gemm(dy, w, b_mn=True) if use_native(dy) else torch.matmul(dy, w)


def _wgrad(dy, x, w):
    """dW (+)= dyᵀ x into ``w.main_grad`` when the engine provides one; returns the gradient tensor otherwise."""
    from verl_b200.ops.functional import gemm, use_native

    mg = getattr(w, "main_grad", None)
    if use_native(dy):
        if mg is not None:
            gemm(dy, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
            return None
        return gemm(dy, x, a_mn=True, b_mn=True)
    dw = dy.float().t() @ x.float()
    if mg is not None:
        mg.add_(dw.to(mg.dtype))
        return None
    return dw.to(w.dtype)


class _AllGatherLinear(torch.autograd.Function):
    """y [T, out_local] = all_gather(x_shard) @ wᵀ (+ bias)."""

    @staticmethod
    def forward(ctx, x_shard, w, bias, group, tpctx):
        ctx.save_for_backward(x_shard, w)
        ctx.group, ctx.bias_ref, ctx.tpctx = group, bias, None
        if tpctx is not None and fused_comm_enabled() and x_shard.is_cuda and x_shard.shape[0] % 128 == 0 and \
                x_shard.shape[0] * tpctx.world <= tpctx.max_tokens:
            ctx.tpctx = tpctx
            return tpctx.allgather_linear(x_shard.contiguous(), w, bias)
        return torch.nn.functional.linear(_all_gather_rows(x_shard, group), w, bias)

    @staticmethod
    def backward(ctx, dy):
        x_shard, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = None
        t = ctx.tpctx
        fused = t is not None and dy.shape[0] % t.world == 0 and w.shape[1] % 32 == 0 and (dy.shape[0] // t.world) * w.shape[1] <= t.slot_elems \
            and dy.data_ptr() % 16 == 0
        x_full = work = None
        if ctx.needs_input_grad[1] and fused:
            # the gather of the forward input for the weight gradient runs on NCCL's stream underneath the fused dgrad
            x_full = torch.empty(x_shard.shape[0] * t.world, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
            work = dist.all_gather_into_tensor(x_full, x_shard.contiguous(), group=ctx.group, async_op=True)
        if ctx.needs_input_grad[0]:
            # activation gradient GEMM with the reduce-scatter in its epilogue (rows go straight to their owners' slots)
            dx = t.gemm_reduce_scatter(dy, w, transposed=True) if fused else _reduce_scatter_rows(_dgrad(dy, w), ctx.group)
        dw = None
        if ctx.needs_input_grad[1]:
            if work is not None:
                work.wait()
            dw = _wgrad(dy, x_full if x_full is not None else _all_gather_rows(x_shard, ctx.group), w)
        db = None
        b = ctx.bias_ref
        if b is not None and ctx.needs_input_grad[2]:
            bsum = dy.float().sum(0)
            mg = getattr(b, "main_grad", None)
            if mg is not None:
                mg.add_(bsum.to(mg.dtype))
            else:
                db = bsum.to(b.dtype)
        return dx, dw, db, None, None


class _LinearReduceScatter(torch.autograd.Function):
    """y_shard [T/tp, out] = reduce_scatter(x @ wᵀ) with x [T, in_local], w [out, in_local]."""

    @staticmethod
    def forward(ctx, x, w, group, tpctx):
        ctx.save_for_backward(x, w)
        ctx.group, ctx.tpctx = group, None
        if tpctx is not None and fused_comm_enabled() and x.is_cuda and x.shape[0] % tpctx.world == 0 and w.shape[0] % 32 == 0 and \
                (x.shape[0] // tpctx.world) * w.shape[0] <= tpctx.slot_elems:
            ctx.tpctx = tpctx
            return tpctx.gemm_reduce_scatter(x.contiguous(), w)
        return _reduce_scatter_rows(torch.nn.functional.linear(x, w), group)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        dy_shard = dy_shard.contiguous()
        t = ctx.tpctx
        if t is not None and ctx.needs_input_grad[0] and dy_shard.shape[0] % 128 == 0 and dy_shard.shape[1] == t.hidden and \
                dy_shard.shape[0] * t.world <= t.max_tokens and w.shape[1] % 8 == 0:
            # all-gather of the output gradient fused into the activation-gradient GEMM; the gathered rows stay in the staging
            # buffer and feed the weight gradient, so no separate all-gather runs at all
            dx = t.allgather_linear(dy_shard, w, None, transposed=True)
            dw = _wgrad(t.gathered_operand(dy_shard), x, w) if ctx.needs_input_grad[1] else None
            return dx, dw, None, None
        dy = _all_gather_rows(dy_shard, ctx.group)
        dx = _dgrad(dy, w) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dy, x, w) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def allgather_linear(x_shard, w, bias, group, tpctx=None):
    return _AllGatherLinear.apply(x_shard, w, bias, group, tpctx)


def linear_reduce_scatter(x, w, group, tpctx=None):
    return _LinearReduceScatter.apply(x, w, group, tpctx)
