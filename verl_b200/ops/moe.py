"""Mixture-of-experts block: softmax top-k router (optionally *replaying* forced expert choices), token permutation,
grouped expert SwiGLU MLP, weighted un-permutation; optional expert parallelism through an all-to-all.

The reference gets this from Megatron-Core / TransformerEngine (``moe_token_dispatcher_type: alltoall``,
``verl/workers/engine/megatron/transformer_impl.py:266-267,338-339``) and patches the router for replay
(``verl/utils/megatron/router_replay_patch.py:38-165``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import functional as Fn

__all__ = ["route_topk", "moe_forward", "permute_tokens", "unpermute_tokens", "ep_row_tables", "FusedEPContext"]


def route_topk(logits: torch.Tensor, top_k: int, norm_topk_prob: bool, forced_topk: Optional[torch.Tensor] = None):
    """Softmax over experts, then top-k. With ``forced_topk`` ([T, k] expert ids, −1 = not forced) the recorded choice
    replaces the arg-top-k while the *weights* still come from this forward's probabilities, so gradients reach the
    router exactly as in a normal step (router replay R2/R3)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if forced_topk is not None:
        f = forced_topk.to(idx.device).long()
        use = (f >= 0).all(dim=-1, keepdim=True)
        idx = torch.where(use, f.clamp(min=0), idx)
        w = torch.gather(probs, -1, idx)
    if norm_topk_prob:
        w = w / w.sum(dim=-1, keepdim=True).clamp_min(1e-20)
    return w, idx, probs


def permute_tokens(x: torch.Tensor, idx: torch.Tensor, num_experts: int):
    """Replicate each token once per chosen expert and sort the copies by expert id.
    Returns (permuted [T·k, H], order [T·k] = source row in the flattened (token, slot) space, tokens_per_expert [E])."""
    T, k = idx.shape
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return x.index_select(0, order // k), order, counts


def unpermute_tokens(y: torch.Tensor, order: torch.Tensor, weights: torch.Tensor, T: int) -> torch.Tensor:
    k = weights.shape[1]
    w = weights.reshape(-1).index_select(0, order).to(y.dtype)
    out = torch.zeros(T, y.shape[1], dtype=y.dtype, device=y.device)
    out.index_add_(0, order // k, y * w[:, None])
    return out


GROUP_BLOCK = 128


def padded_layout(counts: torch.Tensor, n_rows: int, block: int = GROUP_BLOCK):
    """For rows sorted by expert (``counts[e]`` rows each): destination row of every sorted row in a layout where each
    expert's segment is padded to a multiple of ``block`` rows, plus the tables the grouped GEMM kernels take. Everything
    stays on the device; the padded size is the static upper bound ``ceil((n + E·(block−1)) / block)·block``.
    Returns (dest [n] int64, R, blk_expert [R/block] int32 (−1 = unused), expert_rng [E, 2] int32 block ranges)."""
    E = counts.numel()
    dev = counts.device
    padded = (counts + block - 1) // block * block
    pad_end = torch.cumsum(padded, 0)
    pad_off = pad_end - padded
    off = torch.cumsum(counts, 0) - counts
    sorted_e = torch.repeat_interleave(torch.arange(E, device=dev), counts, output_size=n_rows)
    dest = pad_off[sorted_e] + (torch.arange(n_rows, device=dev) - off[sorted_e])
    R = (n_rows + E * (block - 1) + block - 1) // block * block
    starts = torch.arange(R // block, device=dev) * block
    be = torch.searchsorted(pad_end, starts, right=True)
    blk_expert = torch.where(starts < pad_end[-1], be, torch.full_like(be, -1)).to(torch.int32)
    rng = torch.stack([pad_off // block, pad_end // block], 1).to(torch.int32).contiguous()
    return dest, R, blk_expert, rng


class _GroupedLinear(torch.autograd.Function):
    """y[rows of expert e] = x[rows] @ w[e]ᵀ for row blocks sorted and padded per expert (one kernel for all experts)."""

    @staticmethod
    def forward(ctx, x, w, blk_expert, expert_rng):
        from . import _ext

        ctx.save_for_backward(x, w, blk_expert, expert_rng)
        return _ext.ops().gemm_grouped(x.contiguous(), w, blk_expert, False)

    @staticmethod
    def backward(ctx, dy):
        from . import _ext

        x, w, blk_expert, expert_rng = ctx.saved_tensors
        o = _ext.ops()
        dy = dy.contiguous()
        dx = o.gemm_grouped(dy, w, blk_expert, True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                o.gemm_grouped_wgrad(dy, x, expert_rng, mg, True)
            else:
                dw = torch.zeros_like(w)
                o.gemm_grouped_wgrad(dy, x, expert_rng, dw, False)
        return dx, dw, None, None


def _experts_grouped(xp: torch.Tensor, counts: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """Same contract as ``_experts_local`` on the sm_100a grouped GEMM: three launches per layer instead of 2·E."""
    n = xp.shape[0]
    dest, R, blk_expert, rng = padded_layout(counts, n)
    xpad = torch.zeros(R, xp.shape[1], dtype=xp.dtype, device=xp.device).index_copy(0, dest, xp)
    h = Fn.swiglu(_GroupedLinear.apply(xpad, gate_up, blk_expert, rng))
    y = _GroupedLinear.apply(h, down, blk_expert, rng)
    return y.index_select(0, dest)


def _experts_local(xp: torch.Tensor, counts: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, first_expert: int = 0):
    """Grouped SwiGLU MLP over rows already sorted by (local) expert."""
    if Fn.use_native(xp) and gate_up.shape[1] % 8 == 0 and xp.shape[1] % 128 == 0 and gate_up.shape[1] % 256 == 0 and xp.shape[0] > 0:
        return _experts_grouped(xp, counts, gate_up, down)
    out = torch.empty(xp.shape[0], down.shape[1], dtype=xp.dtype, device=xp.device)
    start = 0
    for e, n in enumerate(counts.tolist()):
        if n == 0:
            continue
        seg = xp[start : start + n]
        h = Fn.swiglu(Fn.linear(seg, gate_up[e]))
        out[start : start + n] = Fn.linear(h, down[e])
        start += n
    return out


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all over rows; backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, send_splits, recv_splits, group):
        ctx.group, ctx.send, ctx.recv = group, send_splits, recv_splits
        out = x.new_empty(sum(recv_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty(sum(ctx.send), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return out, None, None, None


# ---------------------------------------------------------------------------------------------------------------------
# Expert parallelism with dispatch and combine fused into the grouped GEMMs (sm_100a, peers reachable over NVLink).
#   dispatch: the gate/up grouped GEMM fetches every operand row from the rank that holds the token (copy warps gather 128-row
#             blocks into local staging while the tensor cores multiply blocks that have arrived) — no all-to-all, no permuted copy;
#   combine:  the down-projection grouped GEMM's epilogue multiplies each output row by its routing weight and stores it into the
#             token owner's [top_k, T, H] slot buffer; the owner sums its k slots.
# The backward pass uses the same two kernels in the other direction (gradient rows are gathered from the token owners by the
# dispatch kernel fused with the down-projection's input-gradient GEMM; input gradients go back through the combine epilogue).
# Reference: Megatron-Core's alltoall token dispatcher (verl/workers/engine/megatron/transformer_impl.py:266-267,338-339).
def ep_row_tables(idx_all: torch.Tensor, w_all: torch.Tensor, rank: int, e_local: int):
    """Routing of ALL ranks' tokens → the row tables of this rank's grouped GEMMs.
    ``idx_all`` [W, Tc, k] expert ids (−1: no such token), ``w_all`` [W, Tc, k] routing weights. Rows are the (token, slot) pairs
    routed to experts ``[rank·e_local, (rank+1)·e_local)``, sorted by expert, every expert padded to a multiple of 128 rows.
    Returns ``row_src`` int32 [R] ((source rank << 24) | token, −1 padding), ``row_dst`` int32 [R] ((source rank << 24) | (slot·Tc +
    token)), ``row_w`` fp32 [R], ``blk_expert`` int32 [R/128], ``expert_rng`` int32 [e_local, 2]."""
    W, Tc, k = idx_all.shape
    if idx_all.is_cuda:
        from . import _ext

        if _ext.available():      # three launches on the device (csrc/moe_tables.cu) instead of the tensor ops below
            return _ext.ops().ep_row_tables(idx_all.to(torch.int32).contiguous(), w_all.float().contiguous(), int(rank), int(e_local))
    lo = rank * e_local
    dev = idx_all.device
    flat = idx_all.reshape(-1)
    sel = ((flat >= lo) & (flat < lo + e_local)).nonzero(as_tuple=True)[0]          # the one host synchronisation: R is needed for allocation
    n = int(sel.numel())
    le, order = torch.sort(flat.index_select(0, sel) - lo, stable=True)             # local expert of every row, rows grouped by expert
    sel = sel.index_select(0, order)
    counts = torch.zeros(e_local, dtype=torch.long, device=dev).scatter_add_(0, le, torch.ones_like(le))
    # block-padded layout (same as ``padded_layout``, with the sorted expert ids at hand instead of a repeat_interleave)
    padded = (counts + GROUP_BLOCK - 1) // GROUP_BLOCK * GROUP_BLOCK
    pad_end = torch.cumsum(padded, 0)
    pad_off = pad_end - padded
    off = torch.cumsum(counts, 0) - counts
    dest = pad_off[le] + (torch.arange(n, device=dev) - off[le])
    R = (n + e_local * (GROUP_BLOCK - 1) + GROUP_BLOCK - 1) // GROUP_BLOCK * GROUP_BLOCK
    starts = torch.arange(R // GROUP_BLOCK, device=dev) * GROUP_BLOCK
    be = torch.searchsorted(pad_end, starts, right=True)
    blk_expert = torch.where(starts < pad_end[-1], be, torch.full_like(be, -1)).to(torch.int32)
    rng = torch.stack([pad_off // GROUP_BLOCK, pad_end // GROUP_BLOCK], 1).to(torch.int32).contiguous()
    tok_flat = sel // k
    src, token, slot = tok_flat // Tc, tok_flat % Tc, sel % k
    tables = torch.full((2, R), -1, dtype=torch.int32, device=dev)
    tables[:, dest] = torch.stack([(src << 24) | token, (src << 24) | (slot * Tc + token)]).to(torch.int32)
    row_src, row_dst = tables[0], tables[1]
    row_w = torch.zeros(R, dtype=torch.float32, device=dev)
    row_w[dest] = w_all.reshape(-1).index_select(0, sel).float()
    return row_src, row_dst, row_w, blk_expert, rng


class FusedEPContext:
    """Symmetric buffers of one expert-parallel group: ``xbuf`` [max_tokens, H] holds this rank's tokens (forward) or output
    gradients (backward) for the peers to fetch, ``cbuf`` [top_k · max_tokens, H] receives the expert outputs (or input gradients)
    of this rank's tokens, one slot per chosen expert."""

    def __init__(self, group, host_group, max_tokens: int, hidden: int, top_k: int):
        from verl_b200.parallel.symm_mem import SymmetricBuffer

        from . import _ext

        self.group, self.ops = group, _ext.ops()
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_tokens, self.hidden, self.top_k = max_tokens, hidden, top_k
        self.xbuf = SymmetricBuffer(max_tokens * hidden * 2, group, host_group)
        self.cbuf = SymmetricBuffer(top_k * max_tokens * hidden * 2, group, host_group)
        self.calls = 0

    def publish(self, x: torch.Tensor) -> None:
        """Copy ``x`` [T, H] into the symmetric token buffer and wait until every rank has done so."""
        self.xbuf.tensor(torch.bfloat16, x.numel()).view_as(x).copy_(x)
        self.xbuf.barrier()

    def collect(self, T: int, Tc: int) -> torch.Tensor:
        """After every rank's combine GEMM: sum this rank's top_k slots → [T, H]."""
        self.cbuf.barrier()
        out = torch.empty(T, self.hidden, dtype=torch.bfloat16, device=torch.device("cuda", torch.cuda.current_device()))
        self.ops.slots_reduce(self.cbuf.tensor(torch.bfloat16, self.top_k * Tc * self.hidden), self.top_k, Tc * self.hidden, T, self.hidden, None, out)
        return out


class _FusedEPMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, idx, gate_up, down, fctx: FusedEPContext):
        o = fctx.ops
        T, H = x.shape
        k = idx.shape[1]
        W, rank = fctx.world, fctx.rank
        e_local = gate_up.shape[0]
        dev = x.device
        # routing of all ranks (small): token counts differ between ranks, so pad to the largest
        tc = torch.tensor([T], dtype=torch.int64, device=dev)
        dist.all_reduce(tc, op=dist.ReduceOp.MAX, group=fctx.group)
        Tc = int(tc.item())
        assert Tc <= fctx.max_tokens, f"{Tc} tokens exceed the expert-parallel buffers ({fctx.max_tokens})"
        idx_pad = torch.full((Tc, k), -1, dtype=torch.int32, device=dev)
        idx_pad[:T] = idx.to(torch.int32)
        w_pad = torch.zeros(Tc, k, dtype=torch.float32, device=dev)
        w_pad[:T] = w.detach().float()
        idx_all = torch.empty(W, Tc, k, dtype=torch.int32, device=dev)
        w_all = torch.empty(W, Tc, k, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(idx_all, idx_pad, group=fctx.group)
        dist.all_gather_into_tensor(w_all, w_pad, group=fctx.group)
        row_src, row_dst, row_w, blk_expert, rng = ep_row_tables(idx_all, w_all, rank, e_local)
        R = row_src.numel()
        fctx.publish(x.detach().contiguous())
        xg = torch.empty(R, H, dtype=torch.bfloat16, device=dev)          # the gathered operand, written by the kernel
        flags = torch.empty(R // GROUP_BLOCK, dtype=torch.int32, device=dev)
        h = o.gemm_grouped_dispatch(fctx.xbuf.table(), H, row_src, gate_up, blk_expert, xg, flags, False)
        a = o.swiglu_fwd(h)
        o.gemm_grouped_combine(a, down, blk_expert, row_dst, row_w, fctx.cbuf.table(), H, False)
        y = fctx.collect(T, Tc)
        fctx.calls += 1
        ctx.save_for_backward(xg, h, a, gate_up, down, row_src, row_dst, row_w, blk_expert, rng)
        ctx.fctx, ctx.dims = fctx, (T, Tc, k)
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, h, a, gate_up, down, row_src, row_dst, row_w, blk_expert, rng = ctx.saved_tensors
        fctx = ctx.fctx
        o = fctx.ops
        T, Tc, k = ctx.dims
        H = dy.shape[1]
        R = row_src.numel()
        dev = dy.device
        # gradient rows of this rank's experts' outputs live with the token owners: fetch them fused with d(act) = dy_rows @ W_down
        fctx.publish(dy.contiguous())
        dyg = torch.empty(R, H, dtype=torch.bfloat16, device=dev)
        flags = torch.empty(R // GROUP_BLOCK, dtype=torch.int32, device=dev)
        da = o.gemm_grouped_dispatch(fctx.xbuf.table(), H, row_src, down, blk_expert, dyg, flags, True)      # [R, I], not yet weighted
        dw_rows = (da.float() * a.float()).sum(-1)                           # d(loss)/d(routing weight) of every row
        wcol = row_w[:, None]
        da = (da.float() * wcol).to(torch.bfloat16)
        dh = o.swiglu_bwd(h, da)
        dyw = (dyg.float() * wcol).to(torch.bfloat16)
        d_down = d_gate_up = None
        for wt, dy_op, x_op, which in ((down, dyw, a, "down"), (gate_up, dh, xg, "gate_up")):
            mg = getattr(wt, "main_grad", None)
            if mg is not None:
                o.gemm_grouped_wgrad(dy_op, x_op, rng, mg, True)
            else:
                g = torch.zeros_like(wt)
                o.gemm_grouped_wgrad(dy_op, x_op, rng, g, False)
                if which == "down":
                    d_down = g
                else:
                    d_gate_up = g
        # input gradients travel back to the token owners through the combine epilogue (weight 1), k slots per token
        ones = (row_dst >= 0).float()
        o.gemm_grouped_combine(dh, gate_up, blk_expert, row_dst, ones, fctx.cbuf.table(), H, True)
        dx = fctx.collect(T, Tc)
        # routing-weight gradients: a few floats per row, gathered by everyone and picked by the owner
        rc = torch.tensor([R], dtype=torch.int64, device=dev)
        dist.all_reduce(rc, op=dist.ReduceOp.MAX, group=fctx.group)
        Rc = int(rc.item())
        code_l = torch.full((Rc,), -1, dtype=torch.int32, device=dev)
        code_l[:R] = row_dst
        val_l = torch.zeros(Rc, dtype=torch.float32, device=dev)
        val_l[:R] = dw_rows
        code = torch.empty(fctx.world * Rc, dtype=torch.int32, device=dev)
        val = torch.empty(fctx.world * Rc, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(code, code_l, group=fctx.group)
        dist.all_gather_into_tensor(val, val_l, group=fctx.group)
        code = code.long()
        mine = (code >= 0) & ((code >> 24) == fctx.rank)
        dwk = torch.zeros(k * Tc, dtype=torch.float32, device=dev)
        dwk[(code[mine] & 0xFFFFFF)] = val[mine]
        dw = dwk.view(k, Tc).t()[:T].contiguous()
        return dx, dw, None, d_gate_up, d_down, None


def moe_forward(x: torch.Tensor, router_w: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, top_k: int,
                norm_topk_prob: bool = True, forced_topk: Optional[torch.Tensor] = None, ep_group=None, ep_ctx: Optional[FusedEPContext] = None):
    """x [T, H]; router_w [E, H]; gate_up [E_local, 2I, H]; down [E_local, H, I]. Returns (y [T, H], topk_idx [T, k]).
    With ``ep_ctx`` (and bf16 CUDA tensors) the expert-parallel exchange runs inside the grouped GEMMs instead of as all-to-alls."""
    T = x.shape[0]
    E = router_w.shape[0]
    logits = F.linear(x, router_w)
    w, idx, _ = route_topk(logits, top_k, norm_topk_prob, forced_topk)
    if ep_ctx is not None and Fn.use_native(x) and x.shape[1] % 128 == 0 and gate_up.shape[1] % 256 == 0:
        return _FusedEPMoE.apply(x, w, idx, gate_up, down, ep_ctx), idx
    xp, order, counts = permute_tokens(x, idx, E)
    if ep_group is None or dist.get_world_size(ep_group) == 1:
        yp = _experts_local(xp, counts, gate_up, down)
    else:
        ep = dist.get_world_size(ep_group)
        e_local = E // ep
        # dispatch: rows for experts [r*e_local, (r+1)*e_local) go to rank r
        send_counts = counts.reshape(ep, e_local)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=ep_group)
        send_splits = send_counts.sum(1).tolist()
        recv_splits = recv_counts.sum(1).tolist()
        recv = _AllToAllRows.apply(xp, send_splits, recv_splits, ep_group)
        # received rows are grouped by source rank, then by local expert: regroup by local expert
        rc = recv_counts.tolist()
        src_expert = torch.cat([torch.full((rc[s][e],), e, dtype=torch.long) for s in range(ep) for e in range(e_local)]).to(x.device) \
            if recv.shape[0] else torch.zeros(0, dtype=torch.long, device=x.device)
        perm2 = torch.argsort(src_expert, stable=True)
        local_counts = recv_counts.sum(0)
        yl = _experts_local(recv.index_select(0, perm2), local_counts, gate_up, down)
        back = torch.empty_like(yl)
        back[perm2] = yl
        yp = _AllToAllRows.apply(back, recv_splits, send_splits, ep_group)
    y = unpermute_tokens(yp, order, w, T)
    return y, idx
