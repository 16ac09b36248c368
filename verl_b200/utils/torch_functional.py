"""Tensor helpers shared by the algorithms, engines and trainers.

Parity target: ``verl/utils/torch_functional.py`` (logprobs_from_logits :73, entropy_from_logits :231, masked ops
:273-349, get_response_mask :414, LR schedules :765-986, distributed stats :501-687).
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.optim.lr_scheduler import LambdaLR

__all__ = [
    "logprobs_from_logits",
    "entropy_from_logits",
    "entropy_from_logits_with_chunking",
    "calculate_sum_pi_squared_from_logits",
    "masked_sum",
    "masked_mean",
    "masked_var",
    "masked_whiten",
    "clip_by_value",
    "get_response_mask",
    "get_eos_mask",
    "compute_position_id_with_mask",
    "pad_sequence_to_length",
    "pad_2d_list_to_length",
    "postprocess_data",
    "get_constant_schedule_with_warmup",
    "get_cosine_schedule_with_warmup",
    "get_wsd_schedule_with_warmup",
    "allgather_dict_tensors",
    "broadcast_dict_tensor",
    "distributed_mean_max_min_std",
    "distributed_masked_mean",
    "expand_as_nested",
]


# ------------------------------------------------------------------------------------------------ logits → stats
def logprobs_from_logits(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[labels]`` computed without materialising the full log-softmax in fp32 for bf16 inputs."""
    if logits.dtype in (torch.float32, torch.float64):
        picked = torch.gather(logits, -1, labels.unsqueeze(-1)).squeeze(-1)
        return picked - torch.logsumexp(logits, dim=-1)
    out = []
    flat_logits = logits.reshape(-1, logits.shape[-1])
    flat_labels = labels.reshape(-1)
    for i in range(0, flat_logits.shape[0], 4096):
        row = flat_logits[i : i + 4096].float()
        out.append(torch.gather(row, -1, flat_labels[i : i + 4096, None]).squeeze(-1) - torch.logsumexp(row, -1))
    return torch.cat(out).reshape(labels.shape)


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    """H = logsumexp(x) − Σ softmax(x)·x."""
    x = logits.float()
    lse = torch.logsumexp(x, dim=-1)
    return lse - torch.sum(torch.softmax(x, dim=-1) * x, dim=-1)


def entropy_from_logits_with_chunking(logits: torch.Tensor, chunk_size: int = 2048) -> torch.Tensor:
    flat = logits.reshape(-1, logits.shape[-1])
    out = torch.empty(flat.shape[0], device=logits.device, dtype=torch.float32)
    for i in range(0, flat.shape[0], chunk_size):
        out[i : i + chunk_size] = entropy_from_logits(flat[i : i + chunk_size])
    return out.reshape(logits.shape[:-1])


def calculate_sum_pi_squared_from_logits(logits: torch.Tensor) -> torch.Tensor:
    """Σ_v π_v² = exp(lse(2x) − 2·lse(x))."""
    x = logits.float()
    return torch.exp(torch.logsumexp(2.0 * x, dim=-1) - 2.0 * torch.logsumexp(x, dim=-1))


# ------------------------------------------------------------------------------------------------ masked ops
def masked_sum(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    valid = torch.where(mask.bool(), values, torch.zeros_like(values))
    return valid.sum() if axis is None else valid.sum(axis)


def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    s = masked_sum(values, mask, axis)
    return s / (mask.sum(axis) + 1e-8)


def masked_var(values: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    mean = masked_mean(values, mask)
    var = masked_mean((values - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if n == 0:
            raise ValueError("masked_var over an empty mask")
        if n == 1:
            raise ValueError("masked_var with a single element and unbiased=True")
        var = var * (n / (n - 1))
    return var


def masked_whiten(values: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    mean, var = masked_mean(values, mask), masked_var(values, mask)
    out = (values - mean) * torch.rsqrt(var + 1e-8)
    if not shift_mean:
        out = out + mean
    return out


def clip_by_value(x: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    return torch.max(torch.min(x, hi), lo)


# ------------------------------------------------------------------------------------------------ masks / ids
def get_response_mask(response_id: torch.Tensor, eos_token=2, dtype=torch.int64) -> torch.Tensor:
    """1 up to and including the first EOS token of each row, 0 afterwards."""
    eos = [eos_token] if isinstance(eos_token, int) else list(eos_token)
    is_eos = torch.isin(response_id, torch.tensor(eos, device=response_id.device)).long()
    return (torch.cumsum(is_eos, dim=1) - is_eos).eq(0).to(dtype)


get_eos_mask = get_response_mask


def compute_position_id_with_mask(mask: torch.Tensor) -> torch.Tensor:
    return torch.clip(torch.cumsum(mask, dim=-1) - 1, min=0, max=None)


def pad_sequence_to_length(t: torch.Tensor, max_len: int, pad_value, left_pad: bool = False) -> torch.Tensor:
    if t.shape[-1] >= max_len:
        return t
    pad = (max_len - t.shape[-1], 0) if left_pad else (0, max_len - t.shape[-1])
    return F.pad(t, pad, "constant", pad_value)


def pad_2d_list_to_length(rows: list[list[int]], pad_token_id: int, max_length: Optional[int] = None) -> torch.Tensor:
    longest = max((len(r) for r in rows), default=0)
    target = max(longest, max_length or 0)
    return torch.tensor([list(r) + [pad_token_id] * (target - len(r)) for r in rows])


def postprocess_data(input_ids, attention_mask, max_length: int, pad_token_id: int, left_pad=True, truncation="error"):
    """Pad or truncate a [1, L] prompt to ``max_length`` (left/right/middle truncation or error)."""
    L = input_ids.shape[-1]
    if L < max_length:
        input_ids = pad_sequence_to_length(input_ids, max_length, pad_token_id, left_pad)
        attention_mask = pad_sequence_to_length(attention_mask, max_length, 0, left_pad)
    elif L > max_length:
        if truncation == "left":
            input_ids, attention_mask = input_ids[:, -max_length:], attention_mask[:, -max_length:]
        elif truncation == "right":
            input_ids, attention_mask = input_ids[:, :max_length], attention_mask[:, :max_length]
        elif truncation == "middle":
            lh = max_length // 2
            rh = max_length - lh
            input_ids = torch.cat([input_ids[:, :lh], input_ids[:, -rh:]], -1)
            attention_mask = torch.cat([attention_mask[:, :lh], attention_mask[:, -rh:]], -1)
        elif truncation == "error":
            raise NotImplementedError(f"sequence length {L} exceeds max_length {max_length}")
        else:
            raise NotImplementedError(f"unknown truncation method {truncation}")
    return input_ids, attention_mask


# ------------------------------------------------------------------------------------------------ LR schedules
def get_constant_schedule_with_warmup(optimizer, num_warmup_steps: int, last_epoch: int = -1):
    def f(step):
        return min(1.0, float(step) / float(max(1, num_warmup_steps))) if num_warmup_steps > 0 else 1.0

    return LambdaLR(optimizer, f, last_epoch)


def get_cosine_schedule_with_warmup(optimizer, num_warmup_steps, num_training_steps, min_lr_ratio=0.0, num_cycles=0.5,
                                    last_epoch=-1, init_lr_ratio: Optional[float] = None):
    min_lr_ratio = 0.0 if min_lr_ratio is None else min_lr_ratio
    init_lr_ratio = 0.0 if init_lr_ratio is None else init_lr_ratio
    coef, intercept = (1 - min_lr_ratio) * 0.5, (1 + min_lr_ratio) * 0.5

    def f(step):
        if step < num_warmup_steps:
            return init_lr_ratio + (1.0 - init_lr_ratio) * (float(step) / float(max(1, num_warmup_steps)))
        prog = float(step - num_warmup_steps) / float(max(1, num_training_steps - num_warmup_steps))
        return max(min_lr_ratio, math.cos(math.pi * float(num_cycles) * 2.0 * prog) * coef + intercept)

    return LambdaLR(optimizer, f, last_epoch)


def get_wsd_schedule_with_warmup(optimizer, num_warmup_steps, num_training_steps, min_lr_ratio=0.0, num_cycles=0.5,
                                 last_epoch=-1, stable_ratio=0.9):
    remaining = max(0, num_training_steps - num_warmup_steps)
    n_stable = int(remaining * stable_ratio)
    n_decay = remaining - n_stable

    def f(step):
        if step < num_warmup_steps:
            return float(step) / float(max(1, num_warmup_steps))
        if step < num_warmup_steps + n_stable:
            return 1.0
        if step < num_training_steps:
            prog = float(step - num_warmup_steps - n_stable) / float(max(1, n_decay))
            return (1.0 - min_lr_ratio) * max(0.0, 0.5 * (1.0 + math.cos(math.pi * float(num_cycles) * 2.0 * prog))) + min_lr_ratio
        return min_lr_ratio

    return LambdaLR(optimizer, f, last_epoch)


# ------------------------------------------------------------------------------------------------ distributed
def allgather_dict_tensors(tensors: dict, size: int, group, dim: int = 0) -> dict:
    out = {}
    for k in sorted(tensors.keys()):
        v = tensors[k]
        bufs = [torch.empty_like(v) for _ in range(size)]
        dist.all_gather(bufs, v.contiguous(), group=group)
        out[k] = torch.cat(bufs, dim=dim)
    return out


def broadcast_dict_tensor(tensors: dict, src: int, group) -> None:
    for k in sorted(tensors.keys()):
        dist.broadcast(tensors[k], src=src, group=group, async_op=False)


def distributed_mean_max_min_std(local: torch.Tensor, compute_max=True, compute_min=True, compute_std=True):
    n = torch.tensor(local.numel(), device=local.device, dtype=torch.float64)
    s = local.double().sum()
    if dist.is_initialized():
        dist.all_reduce(n)
        dist.all_reduce(s)
    mean = (s / n).float()
    mx = mn = std = None
    if compute_max:
        mx = local.max().clone()
        if dist.is_initialized():
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    if compute_min:
        mn = local.min().clone()
        if dist.is_initialized():
            dist.all_reduce(mn, op=dist.ReduceOp.MIN)
    if compute_std:
        sq = ((local.double() - mean.double()) ** 2).sum()
        if dist.is_initialized():
            dist.all_reduce(sq)
        std = torch.sqrt(sq / (n - 1)).float()
    return mean, mx, mn, std


def distributed_masked_mean(local: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    s = (local * mask).sum()
    n = mask.sum().to(s.dtype)
    if dist.is_initialized():
        dist.all_reduce(s)
        dist.all_reduce(n)
    return s / n


def expand_as_nested(per_row: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
    """Broadcast one value per sequence to every token of a packed (jagged) layout."""
    return torch.repeat_interleave(per_row, lengths.to(per_row.device), dim=0)
