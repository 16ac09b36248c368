"""Score centering: a control-variate term that corrects policy gradients for the mismatch between the sampler's and
the trainer's token distributions using only the sampler's top-k head.

The rollout returns, per generated token, the ids and log-probs of its k most likely tokens (the head H). The trainer
evaluates its own log-probs p on the same ids. The sampler's tail is modelled as the trainer's tail rescaled to the
sampler's tail mass, ρ = (1 − q(H)) / (1 − p(H)), which gives the per-token term

    c = Σ_{j∈H} sg[ q_j · w(p_j / q_j) − α · p_j ] · log p_j,      α = ρ · w(1/ρ),

to be subtracted from the policy-gradient loss; ``w`` is the importance-weight rule (none, truncated "TIS", or banded
"IcePop"). Reference: ``verl/trainer/ppo/score_centering.py:35-300``.
"""

from __future__ import annotations

import math
from typing import Callable, Optional

import torch

__all__ = ["dummy_rollout_topk", "pad_rollout_topk", "topk_log_probs_from_logits", "topk_log_probs_from_hidden", "score_centering_weight_fn",
           "score_centering_correction"]

CHUNK = 4096


def dummy_rollout_topk(num_rows: int, k: int, device=None):
    """Uniform head for rows the loss masks out (prompt / padding positions)."""
    ids = torch.arange(k, dtype=torch.int32, device=device).expand(num_rows, k).clone()
    return ids, torch.full((num_rows, k), -math.log(k), dtype=torch.float32, device=device)


def pad_rollout_topk(response_topk_ids, response_topk_log_probs, prompt_length: int):
    """Place the response heads on the packed prompt+response rows: response token r is predicted by row
    ``prompt_length − 1 + r``; all other rows get the dummy head."""
    ids = torch.as_tensor(response_topk_ids)
    lps = torch.as_tensor(response_topk_log_probs, dtype=torch.float32)
    R, k = ids.shape
    total = prompt_length + R
    out_ids, out_lps = dummy_rollout_topk(total, k, ids.device)
    out_ids[prompt_length - 1: prompt_length - 1 + R] = ids.to(torch.int32)
    out_lps[prompt_length - 1: prompt_length - 1 + R] = lps
    return out_ids, out_lps


class _TopKLogProbs(torch.autograd.Function):
    """log_softmax(logits)[ids] with the normaliser recomputed per row chunk in forward and backward."""

    @staticmethod
    def forward(ctx, logits, ids, chunk):
        out = torch.empty(ids.shape, dtype=torch.float32, device=logits.device)
        for s in range(0, logits.shape[0], chunk):
            x = logits[s: s + chunk].float()
            out[s: s + chunk] = x.gather(-1, ids[s: s + chunk]) - torch.logsumexp(x, -1, keepdim=True)
        ctx.save_for_backward(logits, ids)
        ctx.chunk = chunk
        return out

    @staticmethod
    def backward(ctx, g):
        logits, ids = ctx.saved_tensors
        grad = torch.empty_like(logits)
        for s in range(0, logits.shape[0], ctx.chunk):
            x = logits[s: s + ctx.chunk].float()
            gs = g[s: s + ctx.chunk].float()
            d = -torch.softmax(x, -1) * gs.sum(-1, keepdim=True)
            d.scatter_add_(-1, ids[s: s + ctx.chunk], gs)
            grad[s: s + ctx.chunk] = d.to(logits.dtype)
        return grad, None, None


def topk_log_probs_from_logits(logits: torch.Tensor, token_ids: torch.Tensor, chunk_size: int = CHUNK) -> torch.Tensor:
    return _TopKLogProbs.apply(logits, token_ids.long(), chunk_size)


def topk_log_probs_from_hidden(h: torch.Tensor, w: torch.Tensor, token_ids: torch.Tensor, temperature: float = 1.0,
                               chunk_size: int = 1024) -> torch.Tensor:
    """Same from hidden states: logits exist only for ``chunk_size`` rows at a time (recomputed in backward)."""
    from torch.utils.checkpoint import checkpoint

    def f(hc, idc):
        x = (hc @ w.t()).float() / temperature
        return x.gather(-1, idc) - torch.logsumexp(x, -1, keepdim=True)

    ids = token_ids.long()
    parts = [checkpoint(f, h[s: s + chunk_size], ids[s: s + chunk_size], use_reentrant=False) if torch.is_grad_enabled() else
             f(h[s: s + chunk_size], ids[s: s + chunk_size]) for s in range(0, h.shape[0], chunk_size)]
    return torch.cat(parts, 0)


def _parse_threshold(th) -> tuple[float, Optional[float]]:
    """``2.0`` / ``"2.0"`` → (upper, None); ``"0.5_2.0"`` → (upper, lower)."""
    if isinstance(th, str) and "_" in th:
        lo, hi = th.split("_", 1)
        return float(hi), float(lo)
    return float(th), None


def score_centering_weight_fn(rollout_is: Optional[str], rollout_is_threshold=2.0) -> Callable[[torch.Tensor], torch.Tensor]:
    if rollout_is is None:
        return torch.ones_like
    upper, lower = _parse_threshold(rollout_is_threshold)
    if lower is None:
        return lambda r: r.clamp(max=upper)
    return lambda r: torch.where((r >= lower) & (r <= upper), r, torch.zeros_like(r))


def score_centering_correction(train_head_log_probs: torch.Tensor, sampler_head_log_probs: torch.Tensor,
                               weight_fn: Callable[[torch.Tensor], torch.Tensor], eps: float = 1e-6):
    """→ (correction [N] with gradient to the trainer's log-probs, sampler head mass [N], trainer head mass [N])."""
    lp = train_head_log_probs.float()
    lq = sampler_head_log_probs.float()
    with torch.no_grad():
        p, q = lp.exp(), lq.exp()
        p_mass, q_mass = p.sum(-1), q.sum(-1)
        rho = (1 - q_mass).clamp_min(eps) / (1 - p_mass).clamp_min(eps)
        alpha = rho * weight_fn(1.0 / rho)
        coeff = q * weight_fn((lp - lq).exp()) - alpha.unsqueeze(-1) * p
    return (coeff * lp).sum(-1), q_mass, p_mass
