"""Python front-end of the tcgen05 attention kernels: work-list construction + autograd wiring."""

from __future__ import annotations

from functools import lru_cache
from typing import Optional

import torch

from . import _ext

__all__ = ["flash_attention_varlen", "paged_decode_attention", "build_tile_tables"]


@lru_cache(maxsize=64)
def _tile_tables_cached(lens: tuple, q_starts: tuple, device_str: str):
    fwd, bwd = [], []
    tok = 0
    for L, qs in zip(lens, q_starts):
        n = (L + 127) // 128
        q0 = min(qs // 128, n)        # first query tile with real queries (0 unless context parallel)
        for i in range(n):
            # forward tile i of a sequence touches i+1 kv tiles; backward kv tile i is visited by the query tiles at or below it
            if i >= q0:
                fwd.append((i + 1, (tok + i * 128, i * 128, tok, L)))
            bwd.append((n - max(i, q0), (tok + i * 128, i * 128, tok, L, q0, 0, 0, 0)))
        tok += L
    fwd.sort(key=lambda t: -t[0])
    bwd.sort(key=lambda t: -t[0])
    dev = torch.device(device_str)
    ft = torch.tensor([t[1] for t in fwd], dtype=torch.int32).reshape(-1, 4).to(dev, non_blocking=True)
    bt = torch.tensor([t[1] for t in bwd], dtype=torch.int32).reshape(-1, 8).to(dev, non_blocking=True)
    return ft, bt


def build_tile_tables(cu_seqlens_cpu: torch.Tensor, device, q_starts=None) -> tuple[torch.Tensor, torch.Tensor]:
    """Work lists (heaviest first) for the forward (per 128-row query tile) and backward (per 128-row kv tile).

    ``q_starts[s]`` (context parallelism): rows before it in sequence ``s`` carry only keys/values — no forward tile is
    emitted for query tiles that lie entirely before it and the backward skips them; their output rows are undefined."""
    cs = cu_seqlens_cpu.tolist()
    lens = tuple(cs[i + 1] - cs[i] for i in range(len(cs) - 1))
    qs = tuple(int(x) for x in q_starts) if q_starts is not None else (0,) * len(lens)
    return _tile_tables_cached(lens, qs, str(device))


class _FlashVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, fwd_tiles, bwd_tiles, n_heads, n_kv_heads, scale):
        out, lse = _ext.ops().attn_varlen_fwd(qkv, fwd_tiles, n_heads, n_kv_heads, scale)
        ctx.save_for_backward(qkv, out, lse, bwd_tiles)
        ctx.cfg = (n_heads, n_kv_heads, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, bwd_tiles = ctx.saved_tensors
        n_heads, n_kv_heads, scale = ctx.cfg
        dqkv = _ext.ops().attn_varlen_bwd(qkv, out, dout.contiguous(), lse, bwd_tiles, n_heads, n_kv_heads, scale)
        return dqkv, None, None, None, None, None


def flash_attention_varlen(qkv: torch.Tensor, cu_seqlens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                           max_seqlen: int, scale: float, cu_seqlens_cpu: Optional[torch.Tensor] = None, q_starts=None) -> torch.Tensor:
    assert head_dim == 128, "the sm_100a attention kernels are specialised for head_dim 128"
    if cu_seqlens_cpu is None:
        cu_seqlens_cpu = cu_seqlens.cpu()
    ft, bt = build_tile_tables(cu_seqlens_cpu, qkv.device, q_starts)
    if qkv.stride(1) != 1:
        qkv = qkv.contiguous()
    return _FlashVarlen.apply(qkv, ft, bt, n_heads, n_kv_heads, scale)


def paged_decode_attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, kv_lens: torch.Tensor,
                           scale: float, num_splits: int = 1, max_kv_len: int = 0, workspace: Optional[torch.Tensor] = None,
                           out: Optional[torch.Tensor] = None, impl: int = 0) -> torch.Tensor:
    """One query token per sequence against a paged KV cache layer [num_blocks, 2, Hkv, 64, 128]."""
    if out is None:
        out = torch.empty_like(q)
    if q.is_cuda and q.dtype == torch.bfloat16 and _ext.available():
        _ext.ops().attn_paged_decode(q, cache, block_table, kv_lens, out, scale, num_splits, max_kv_len, workspace, impl)
        return out
    return paged_decode_attention_ref(q, cache, block_table, kv_lens, scale, out)


def paged_decode_attention_ref(q, cache, block_table, kv_lens, scale, out=None):
    """PyTorch oracle: gathers each sequence's blocks and runs dense attention."""
    B = q.shape[0]
    nb, _, Hkv, bs, D = cache.shape
    Hq = q.shape[1] // D
    G = Hq // Hkv
    res = torch.empty_like(q) if out is None else out
    for b in range(B):
        L = int(kv_lens[b])
        if L == 0:
            res[b] = 0
            continue
        nblk = (L + bs - 1) // bs
        blocks = block_table[b, :nblk].long()
        k = cache[blocks, 0].permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :L].float()
        v = cache[blocks, 1].permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :L].float()
        qb = q[b].reshape(Hkv, G, D).float()
        att = torch.softmax(torch.einsum("hgd,hld->hgl", qb, k) * scale, dim=-1)
        res[b] = torch.einsum("hgl,hld->hgd", att, v).reshape(Hq * D).to(q.dtype)
    return res
