"""Padding ↔ packing conversions without flash-attn's helpers (reference: ``verl/utils/attention_padding_utils.py:28-105``
re-implements ``unpad_input / pad_input / index_first_axis`` as gather / scatter autograd functions)."""

from __future__ import annotations

import torch
import torch.nn.functional as F

__all__ = ["index_first_axis", "index_put_first_axis", "unpad_input", "pad_input"]


class _IndexFirstAxis(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, indices):
        ctx.save_for_backward(indices)
        ctx.first = x.shape[0]
        return x.index_select(0, indices)

    @staticmethod
    def backward(ctx, g):
        (indices,) = ctx.saved_tensors
        out = torch.zeros(ctx.first, *g.shape[1:], dtype=g.dtype, device=g.device)
        out.index_add_(0, indices, g)
        return out, None


class _IndexPutFirstAxis(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, indices, first):
        ctx.save_for_backward(indices)
        out = torch.zeros(first, *values.shape[1:], dtype=values.dtype, device=values.device)
        out[indices] = values
        return out

    @staticmethod
    def backward(ctx, g):
        (indices,) = ctx.saved_tensors
        return g.index_select(0, indices), None, None


index_first_axis = _IndexFirstAxis.apply
index_put_first_axis = _IndexPutFirstAxis.apply


def unpad_input(hidden_states: torch.Tensor, attention_mask: torch.Tensor):
    """``[B, S, ...]`` + mask → (``[T, ...]``, indices, cu_seqlens int32, max_seqlen, seqlens)."""
    seqlens = attention_mask.sum(-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    cu = F.pad(torch.cumsum(seqlens, 0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape(-1, *hidden_states.shape[2:])
    return index_first_axis(flat, indices), indices, cu, int(seqlens.max()) if seqlens.numel() else 0, seqlens


def pad_input(hidden_states: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    out = index_put_first_axis(hidden_states, indices, batch * seqlen)
    return out.reshape(batch, seqlen, *hidden_states.shape[1:])
