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

__all__ = ["route_topk", "moe_forward", "permute_tokens", "unpermute_tokens"]


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


def moe_forward(x: torch.Tensor, router_w: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, top_k: int,
                norm_topk_prob: bool = True, forced_topk: Optional[torch.Tensor] = None, ep_group=None):
    """x [T, H]; router_w [E, H]; gate_up [E_local, 2I, H]; down [E_local, H, I]. Returns (y [T, H], topk_idx [T, k])."""
    T = x.shape[0]
    E = router_w.shape[0]
    logits = F.linear(x, router_w)
    w, idx, _ = route_topk(logits, top_k, norm_topk_prob, forced_topk)
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
