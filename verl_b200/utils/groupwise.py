"""Group-wise statistics over a flat batch keyed by group id (reference: ``verl/utils/groupwise.py``)."""

from __future__ import annotations

import numpy as np
import torch

__all__ = ["as_torch_index", "group_mean_std"]


def as_torch_index(index, device=None) -> torch.Tensor:
    """Arbitrary hashable group ids (uids, strings) → dense int64 ids, first-occurrence order."""
    if isinstance(index, torch.Tensor):
        _, inv = torch.unique(index, return_inverse=True)
        return inv.to(device or index.device)
    table: dict = {}
    ids = [table.setdefault(x if not isinstance(x, np.generic) else x.item(), len(table)) for x in list(index)]
    return torch.tensor(ids, dtype=torch.int64, device=device)


def group_mean_std(scores: torch.Tensor, gidx: torch.Tensor, eps: float = 1e-6, unbiased: bool = True):
    """Per-group mean and std; singleton groups get mean 0 / std 1 (so their advantage is the raw score)."""
    g = int(gidx.max()) + 1 if gidx.numel() else 0
    s = scores.float()
    cnt = torch.zeros(g, device=s.device).index_add_(0, gidx, torch.ones_like(s))
    sm = torch.zeros(g, device=s.device).index_add_(0, gidx, s)
    sq = torch.zeros(g, device=s.device).index_add_(0, gidx, s * s)
    mean = sm / cnt.clamp_min(1)
    denom = (cnt - 1).clamp_min(1) if unbiased else cnt.clamp_min(1)
    var = ((sq - cnt * mean * mean) / denom).clamp_min(0)
    std = var.sqrt()
    single = cnt <= 1
    mean = torch.where(single, torch.zeros_like(mean), mean)
    std = torch.where(single, torch.ones_like(std), std)
    return mean, std, cnt
