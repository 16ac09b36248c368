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


def _experts_local(xp: torch.Tensor, counts: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, first_expert: int = 0):
    """Grouped SwiGLU MLP over rows already sorted by (local) expert."""
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
