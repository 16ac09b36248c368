"""Prefix sharing for group sampling: the n responses of one prompt reuse ONE forward/backward of the prompt tokens.

GRPO-style batches hold every prompt n times. In the packed (varlen) layout of this framework sharing needs no special
attention kernel: the model runs on the *unique* tokens (each prompt once, every response), and only around the attention
kernel the rows are expanded to full sequences with a gather (``qkv[expand]``) and reduced back with a second gather
(``out[back]``); autograd's scatter-add of the first gather sums the n responses' gradients into the shared prompt
keys/values. All GEMMs, norms and the MLP see ``P + n·R`` instead of ``n·(P + R)`` tokens per group.

The reference reaches the same goal with the external ``prefix_grouper`` attention wrapper
(``verl/trainer/ppo/prefix_grouper_utils.py:23-150``, ``verl/models/transformers/monkey_patch.py:40-72``) and keeps the
samples of one prompt together when it balances batches (``verl/trainer/ppo/ray_trainer.py:1185-1240``).
"""

from __future__ import annotations

from typing import Optional

import torch

__all__ = ["prompt_groups", "SharedPack", "build_shared_pack", "group_preserving_micro_batches", "expand_rows", "select_rows"]


def prompt_groups(input_ids: torch.Tensor, attention_mask: torch.Tensor, prompt_len: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Rows with identical (masked) prompt tokens form a group.

    Returns ``(group_id [bs], first_row [bs])`` where ``first_row[i]`` is the smallest row index of ``i``'s group."""
    bs = input_ids.shape[0]
    p = input_ids[:, :prompt_len] * attention_mask[:, :prompt_len].to(input_ids.dtype)
    key = torch.cat([p, attention_mask[:, :prompt_len].to(p.dtype)], dim=1)      # a masked id 0 is not a real id 0
    _, inv = torch.unique(key, dim=0, return_inverse=True)
    rows = torch.arange(bs, device=input_ids.device)
    first = torch.full((int(inv.max()) + 1 if bs else 0,), bs, dtype=rows.dtype, device=rows.device)
    first.scatter_reduce_(0, inv, rows, reduce="amin")
    return inv, first[inv]


class _ExpandRows(torch.autograd.Function):
    """``x[idx]`` for an index with repeats. Backward sums the gradients of all copies of a row in one pass over a
    (order, offsets) list — one CTA per source row on the GPU kernel, no atomics — instead of an atomic scatter-add."""

    @staticmethod
    def forward(ctx, x, idx, order, offsets):
        ctx.save_for_backward(idx, order, offsets)
        ctx.n = x.shape[0]
        return x.index_select(0, idx)

    @staticmethod
    def backward(ctx, g):
        idx, order, offsets = ctx.saved_tensors
        from verl_b200.ops import _ext

        if g.is_cuda and g.dtype == torch.bfloat16 and _ext.available() and g.shape[1] % 8 == 0:
            return _ext.ops().segment_sum_rows(g.contiguous(), order, offsets), None, None, None
        return torch.zeros(ctx.n, *g.shape[1:], dtype=g.dtype, device=g.device).index_add_(0, idx, g), None, None, None


class _SelectRows(torch.autograd.Function):
    """``x[idx]`` for an index WITHOUT repeats: the backward is a plain row copy into zeros."""

    @staticmethod
    def forward(ctx, x, idx):
        ctx.save_for_backward(idx)
        ctx.n = x.shape[0]
        return x.index_select(0, idx)

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        return torch.zeros(ctx.n, *g.shape[1:], dtype=g.dtype, device=g.device).index_copy_(0, idx, g), None


def expand_rows(x: torch.Tensor, expand: torch.Tensor, order: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    return _ExpandRows.apply(x, expand, order, offsets)


def select_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return _SelectRows.apply(x, idx)


class SharedPack:
    """Index tensors of one prefix-shared micro-batch.

    ``keep``      [bs, L] bool   tokens that exist in the unique layout (all responses; the prompt of a group's first row)
    ``expand``    [E] int64      unique-layout row of every token of the full (per-sequence) layout
    ``back``      [U] int64      full-layout row of every unique token
    """

    __slots__ = ("keep", "expand", "back", "n_unique", "n_full", "order", "offsets")

    def __init__(self, keep, expand, back):
        self.keep, self.expand, self.back = keep, expand, back
        self.n_unique, self.n_full = int(back.numel()), int(expand.numel())
        # copies of every unique row, grouped: order[offsets[u]:offsets[u+1]] are the full-layout rows that read unique row u
        self.order = torch.argsort(expand, stable=True)
        self.offsets = torch.zeros(self.n_unique + 1, dtype=torch.int64, device=expand.device)
        self.offsets[1:] = torch.cumsum(torch.bincount(expand, minlength=self.n_unique), 0)


def build_shared_pack(attention_mask: torch.Tensor, prompt_len: int, first_row: torch.Tensor) -> SharedPack:
    """``attention_mask`` [bs, L] (prompt columns ``[0, prompt_len)`` then response columns), ``first_row`` from
    :func:`prompt_groups`. Unique tokens are ordered row-major; the full layout is the usual packed order of ``attention_mask``."""
    att = attention_mask.bool()
    bs, L = att.shape
    rows = torch.arange(bs, device=att.device)
    is_first = first_row == rows
    col_is_resp = torch.arange(L, device=att.device) >= prompt_len
    own = col_is_resp[None, :] | is_first[:, None]                 # token is stored by its own row
    keep = att & own
    uidx = (torch.cumsum(keep.reshape(-1).to(torch.int64), 0) - 1).reshape(bs, L)
    src = torch.where(own, uidx, uidx.index_select(0, first_row))  # prompt tokens of later rows read the first row's copy
    expand = src[att]
    eidx = (torch.cumsum(att.reshape(-1).to(torch.int64), 0) - 1).reshape(bs, L)
    back = eidx[keep]
    return SharedPack(keep, expand, back)


def group_preserving_micro_batches(resp_lens, prompt_lens, group_ids, max_tokens: int, num_micro_batches: Optional[int] = None) -> list[list[int]]:
    """Micro-batches (lists of row indices) of at most ``max_tokens`` UNIQUE tokens with the rows of a group adjacent.

    Rows are walked group by group; a group that does not fit into what is left of the current micro-batch continues in
    the next one (which stores the prompt again). ``num_micro_batches`` (e.g. the maximum over data-parallel ranks) forces
    at least that many by halving the largest ones."""
    resp_lens, prompt_lens, group_ids = [list(map(int, x)) for x in (resp_lens, prompt_lens, group_ids)]
    order = sorted(range(len(group_ids)), key=lambda i: (group_ids[i], i))
    out: list[list[int]] = []
    cur: list[int] = []
    cur_tokens, cur_groups = 0, set()
    for i in order:
        cost = resp_lens[i] + (0 if group_ids[i] in cur_groups else prompt_lens[i])
        if cur and cur_tokens + cost > max_tokens:
            out.append(cur)
            cur, cur_tokens, cur_groups = [], 0, set()
            cost = resp_lens[i] + prompt_lens[i]
        assert cost <= max_tokens, f"token budget {max_tokens} is smaller than one sequence ({cost} tokens)"
        cur.append(i)
        cur_tokens += cost
        cur_groups.add(group_ids[i])
    if cur:
        out.append(cur)
    if num_micro_batches is not None:
        while len(out) < num_micro_batches:
            k = max(range(len(out)), key=lambda j: len(out[j]))
            if len(out[k]) < 2:
                break
            big = out.pop(k)
            out[k:k] = [big[: len(big) // 2], big[len(big) // 2:]]
    return out
