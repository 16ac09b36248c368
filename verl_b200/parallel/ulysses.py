"""Ulysses sequence parallelism: tokens are sharded over the SP group everywhere except inside attention, where an
all-to-all trades the sequence shard for a head shard (each rank sees the full sequence for ``heads / sp`` heads).

Parity target: ``verl/utils/ulysses.py`` (SeqAllToAll :169-196, gather_seq_scatter_heads :66, gather_heads_scatter_seq
:90, pad/slice :282-334, gather_outputs_and_unpad :247-280) and the attention hook
``verl/models/transformers/monkey_patch.py:87-155`` (KV-head replication when ``sp > n_kv_heads``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

__all__ = ["SeqAllToAll", "gather_seq_scatter_heads", "gather_heads_scatter_seq", "Gather", "ulysses_pad_and_slice_inputs",
           "gather_outputs_and_unpad", "ulysses_attention", "validate_ulysses_config"]


def _a2a(x: torch.Tensor, scatter_dim: int, gather_dim: int, group) -> torch.Tensor:
    ws = dist.get_world_size(group)
    if ws == 1:
        return x
    parts = [t.contiguous() for t in torch.tensor_split(x, ws, dim=scatter_dim)]
    outs = [torch.empty_like(parts[0]) for _ in range(ws)]
    dist.all_to_all(outs, parts, group=group)
    return torch.cat(outs, dim=gather_dim).contiguous()


class SeqAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, x, scatter_dim, gather_dim):
        ctx.group, ctx.scatter_dim, ctx.gather_dim = group, scatter_dim, gather_dim
        return _a2a(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, g):
        return None, _a2a(g, ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None


def gather_seq_scatter_heads(x: torch.Tensor, seq_dim: int, head_dim: int, group, unpadded_dim_size: int = 0) -> torch.Tensor:
    """[.., T/sp, .., H, ..] → [.., T, .., H/sp, ..]"""
    if group is None or dist.get_world_size(group) == 1:
        return x
    x = SeqAllToAll.apply(group, x, head_dim, seq_dim)
    if unpadded_dim_size and unpadded_dim_size % dist.get_world_size(group) != 0:
        x = x.narrow(seq_dim, 0, unpadded_dim_size)
    return x


def gather_heads_scatter_seq(x: torch.Tensor, head_dim: int, seq_dim: int, group) -> torch.Tensor:
    """[.., T, .., H/sp, ..] → [.., T/sp, .., H, ..]"""
    if group is None or dist.get_world_size(group) == 1:
        return x
    sp = dist.get_world_size(group)
    pad = (-x.shape[seq_dim]) % sp
    if pad:
        shape = list(x.shape)
        shape[seq_dim] = pad
        x = torch.cat([x, x.new_zeros(shape)], dim=seq_dim)
    return SeqAllToAll.apply(group, x, seq_dim, head_dim)


class Gather(torch.autograd.Function):
    """all-gather along ``dim`` forward; backward keeps this rank's slice (scaled by sp when ``grad_scaler``)."""

    @staticmethod
    def forward(ctx, group, x, dim, grad_scaler=True):
        ctx.group, ctx.dim, ctx.grad_scaler = group, dim, grad_scaler
        ws, ctx.rank = dist.get_world_size(group), dist.get_rank(group)
        ctx.part = x.shape[dim]
        outs = [torch.empty_like(x) for _ in range(ws)]
        dist.all_gather(outs, x.contiguous(), group=group)
        return torch.cat(outs, dim=dim)

    @staticmethod
    def backward(ctx, g):
        if ctx.grad_scaler:
            g = g * dist.get_world_size(ctx.group)
        return None, g.narrow(ctx.dim, ctx.rank * ctx.part, ctx.part).contiguous(), None, None


def ulysses_pad_and_slice_inputs(input_ids: torch.Tensor, position_ids: Optional[torch.Tensor], sp_size: int, sp_rank: int, dim: int = -1):
    """Pad the packed token axis to a multiple of ``sp_size`` and keep this rank's contiguous slice.
    Returns (ids_slice, pos_slice, pad_size)."""
    T = input_ids.shape[dim]
    pad = (-T) % sp_size
    if pad:
        input_ids = torch.nn.functional.pad(input_ids, (0, pad), value=0)
        if position_ids is not None:
            extra = torch.arange(pad, device=position_ids.device, dtype=position_ids.dtype)
            position_ids = torch.cat([position_ids, extra], dim=dim)
    part = (T + pad) // sp_size
    sl = slice(sp_rank * part, (sp_rank + 1) * part)
    return input_ids[..., sl], (position_ids[..., sl] if position_ids is not None else None), pad


def gather_outputs_and_unpad(x: torch.Tensor, gather_dim: int, unpad_dim: Optional[int] = None, padding_size: int = 0, grad_scaler: bool = True, group=None):
    if group is None or dist.get_world_size(group) == 1:
        return x
    x = Gather.apply(group, x, gather_dim, grad_scaler)
    if unpad_dim is not None and padding_size:
        x = x.narrow(unpad_dim, 0, x.shape[unpad_dim] - padding_size)
    return x


def validate_ulysses_config(num_heads: int, num_kv_heads: int, sp: int):
    assert num_heads % sp == 0, f"num_attention_heads ({num_heads}) must be divisible by ulysses sp size ({sp})"
    assert num_kv_heads % sp == 0 or sp % num_kv_heads == 0, f"kv heads ({num_kv_heads}) and sp size ({sp}) must divide one another"


def ulysses_attention(qkv: torch.Tensor, pb, cfg, group) -> torch.Tensor:
    """Attention on a sequence-sharded fused qkv [T/sp, (Hq+2Hkv)·D]: a2a to [T, (Hq+2Hkv')/sp·D], full-sequence
    attention on the local heads, a2a back to [T/sp, Hq·D]. ``pb`` describes the *global* packed batch."""
    from verl_b200 import ops

    sp = dist.get_world_size(group)
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    validate_ulysses_config(Hq, Hkv, sp)
    Tl = qkv.shape[0]
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    q, k, v = q.reshape(Tl, Hq, D), k.reshape(Tl, Hkv, D), v.reshape(Tl, Hkv, D)
    if Hkv < sp:                       # replicate kv heads so that every rank owns at least one
        rep = sp // Hkv
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    q = gather_seq_scatter_heads(q, 0, 1, group)
    k = gather_seq_scatter_heads(k, 0, 1, group)
    v = gather_seq_scatter_heads(v, 0, 1, group)
    T = int(pb.cu_seqlens_cpu[-1])
    hq_l, hkv_l = q.shape[1], k.shape[1]
    fused = torch.cat([q[:T].reshape(T, -1), k[:T].reshape(T, -1), v[:T].reshape(T, -1)], dim=-1)
    o = ops.attention_varlen(fused, pb.cu_seqlens, hq_l, hkv_l, D, pb.max_seqlen, pb.cu_seqlens_cpu).reshape(T, hq_l, D)
    o = gather_heads_scatter_seq(o, 1, 0, group)
    return o[:Tl].reshape(Tl, Hq * D)
