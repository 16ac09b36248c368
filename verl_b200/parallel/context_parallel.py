"""Context parallelism for packed (varlen) batches: every rank of the group holds a contiguous slice of the packed token
stream; attention all-gathers keys/values and computes this rank's query rows only.

Around the attention kernel the local fused qkv rows are expanded to the sequences that intersect this rank's slice: for each
such sequence the rows from its start up to the end of the slice carry the gathered K/V, the rows of the slice additionally
carry the local Q. The kernels get ``q_starts`` so that query tiles before the slice are neither computed in the forward nor
visited in the backward: a rank does exactly the causal attention work of its own tokens. K/V gradients flow back through
the all-gather as a reduce-scatter. Unlike the head-scattering (Ulysses) scheme this needs no divisibility between heads and
ranks; the price is the causal load imbalance between early and late slices.

Reference: Megatron context parallel through TransformerEngine's ring attention with zig-zag chunks
(``verl/models/mcore/util.py:61-150,236-460``) and its ``contiguous`` layout option; the engine-side input slicing and output
gather are shared with the sequence-parallel path (``verl/utils/ulysses.py:282-334``).
"""

from __future__ import annotations

from functools import lru_cache

import torch
import torch.distributed as dist

__all__ = ["context_parallel_attention", "cp_attention_local", "build_cp_plan", "AllGatherRows"]


class AllGatherRows(torch.autograd.Function):
    """[Tl, C] on every rank → [W·Tl, C] in rank order; backward sums the gradients of all ranks for this rank's rows."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group)
        out = torch.empty(W * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        else:
            parts = list(out.chunk(W, 0))
            dist.all_gather(parts, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group = ctx.group
        W, r = dist.get_world_size(group), dist.get_rank(group)
        g = g.contiguous()
        n = g.shape[0] // W
        if g.is_cuda:
            out = torch.empty(n, *g.shape[1:], dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, group=group)
            return out, None
        dist.all_reduce(g, group=group)           # gloo has no reduce-scatter
        return g[r * n:(r + 1) * n].clone(), None


def zigzag_ranges(t_pad: int, world: int, rank: int) -> list:
    """Zig-zag placement: the stream is cut into ``2·world`` chunks and rank ``r`` takes chunks ``r`` and ``2·world − 1 − r``,
    so every rank holds an early and a late piece and the causal attention work is balanced."""
    c = t_pad // (2 * world)
    return [(rank * c, (rank + 1) * c), ((2 * world - 1 - rank) * c, (2 * world - rank) * c)]


def zigzag_permutation(t_pad: int, world: int) -> torch.Tensor:
    """Global token index of every row of the rank-order concatenation of the zig-zag slices."""
    return torch.cat([torch.arange(a, b) for r in range(world) for a, b in zigzag_ranges(t_pad, world, r)])


@lru_cache(maxsize=64)
def _plan_cached(cu: tuple, t_pad: int, world: int, rank: int, zigzag: bool = False):
    tl = t_pad // world
    ranges = zigzag_ranges(t_pad, world, rank) if zigzag else [(rank * tl, (rank + 1) * tl)]
    seqs = [(cu[i], cu[i + 1]) for i in range(len(cu) - 1) if cu[i + 1] > cu[i]]
    if cu[-1] < t_pad:
        seqs.append((cu[-1], t_pad))                  # padding tokens form a sequence of their own
    kv_idx, q_pos, lens, q_starts = [], [], [], []
    base = 0
    for p0, p1 in ranges:                             # local rows are ordered range by range
        for s0, s1 in seqs:
            if s1 <= p0 or s0 >= p1:
                continue
            e1 = min(s1, p1)
            l0 = max(s0, p0)
            kv_idx.append(torch.arange(s0, e1))
            q_pos.append(torch.arange(base + (l0 - s0), base + (e1 - s0)))
            lens.append(e1 - s0)
            q_starts.append(l0 - s0)
            base += e1 - s0
    cu_exp = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu_exp[1:] = torch.cumsum(torch.tensor(lens), 0)
    return torch.cat(kv_idx), torch.cat(q_pos), cu_exp, tuple(q_starts), max(lens)


def build_cp_plan(cu_seqlens_cpu: torch.Tensor, t_pad: int, world: int, rank: int, zigzag: bool = False):
    """→ (kv_idx [E] global token of every expanded row, q_pos [Tl] expanded row of every local token, cu_exp, q_starts, max_len)."""
    return _plan_cached(tuple(int(x) for x in cu_seqlens_cpu.tolist()), int(t_pad), int(world), int(rank), bool(zigzag))


def context_parallel_attention(qkv: torch.Tensor, pb, cfg, group) -> torch.Tensor:
    """``qkv`` [T/W, (Hq+2Hkv)·D]: this rank's slice of the packed stream (rope already applied); ``pb.cu_seqlens_cpu``
    describes the whole micro-batch. Returns the attention output of the local rows [T/W, Hq·D]."""
    W, r = dist.get_world_size(group), dist.get_rank(group)
    q_size = cfg.num_attention_heads * cfg.head_dim
    kv_all = AllGatherRows.apply(qkv[:, q_size:].contiguous(), group)
    return cp_attention_local(qkv[:, :q_size], kv_all, pb.cu_seqlens_cpu, cfg, W, r, bool(getattr(pb, "cp_zigzag", False)))


def cp_attention_local(q: torch.Tensor, kv_all: torch.Tensor, cu_seqlens_cpu: torch.Tensor, cfg, W: int, r: int, zigzag: bool) -> torch.Tensor:
    """The rank-local part: ``q`` [T/W, Hq·D] are rank ``r``'s query rows, ``kv_all`` [T, 2·Hkv·D] the K/V rows of all ranks in
    rank order (for the zig-zag placement that is the zig-zag order). No communication happens here, so one process can
    play every rank in turn."""
    from verl_b200 import ops

    tl = q.shape[0]
    q_size = cfg.num_attention_heads * cfg.head_dim
    kv_idx, q_pos, cu_exp, q_starts, max_len = build_cp_plan(cu_seqlens_cpu, tl * W, W, r, zigzag)
    dev = q.device
    if zigzag:      # the gathered K/V rows come in rank order = zig-zag order: look global tokens up through the inverse
        kv_idx = torch.argsort(zigzag_permutation(tl * W, W)).index_select(0, kv_idx)
    kv_idx, q_pos = kv_idx.to(dev), q_pos.to(dev)
    q_exp = q.new_zeros(kv_idx.numel(), q_size).index_copy(0, q_pos, q)
    qkv_exp = torch.cat([q_exp, kv_all.index_select(0, kv_idx)], dim=1)
    o = ops.attention_varlen(qkv_exp, cu_exp.to(dev), cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, max_len, cu_exp,
                             q_starts=q_starts)
    return o.index_select(0, q_pos)
