"""Fused RL losses: one kernel for the clipped PPO/GRPO surrogate + KL-to-reference term (value, gradient and logging
statistics), one for the GRPO group-normalised advantage. Both fall back to the PyTorch formulation in
``trainer.ppo.core_algos`` off-GPU; the fused path covers the ``vanilla`` (dual-clip PPO) loss mode.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _ext

__all__ = ["gae_advantage", "fused_value_loss", "agg_weights", "fused_ppo_loss", "fused_ppo_available", "grpo_advantage", "KL_TYPES"]

KL_TYPES = {None: 0, "kl": 1, "k1": 1, "abs": 2, "mse": 3, "k2": 3, "low_var_kl": 4, "k3": 4}


def agg_weights(mask: torch.Tensor, mode: str, dp_size: int = 1, batch_num_tokens=None, global_batch_size=None,
                loss_scale_factor=None) -> torch.Tensor:
    """Per-token weights w with ``Σ w·L == agg_loss(L, mask, mode, ...)`` for every loss matrix L."""
    m = mask.float()
    if mode == "token-mean":
        n = batch_num_tokens if batch_num_tokens is not None else m.sum()
        return m * (dp_size / n)
    if mode == "token-sum":
        return m * float(dp_size)
    ntok = m.sum(-1, keepdim=True)
    alive = (ntok > 0).float()
    g = global_batch_size if global_batch_size is not None else alive.sum()
    if mode in ("seq-mean-token-sum", "seq-mean-token-sum-norm"):
        w = m * alive * (dp_size / g)
        if mode == "seq-mean-token-sum-norm":
            w = w / (loss_scale_factor if loss_scale_factor is not None else mask.shape[-1])
        return w
    if mode == "seq-mean-token-mean":
        return m / (ntok + 1e-8) * alive * (dp_size / g)
    raise ValueError(f"Invalid loss_agg_mode: {mode}")


def fused_ppo_available(log_prob: torch.Tensor) -> bool:
    return log_prob.is_cuda and _ext.available()


class _FusedPPOLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lp, old_lp, ref_lp, adv, weight, mask, is_w, clip_lo, clip_hi, clip_c, kl_type, kl_coef):
        f = lambda t: None if t is None else t.detach().float().contiguous()
        loss, grad, stats = _ext.ops().ppo_loss(f(lp), f(old_lp), f(ref_lp), f(adv), f(weight), f(mask), f(is_w), float(clip_lo), float(clip_hi),
                                                float(clip_c), int(kl_type), float(kl_coef))
        ctx.save_for_backward(grad)
        ctx.lp_dtype = lp.dtype
        ctx.mark_non_differentiable(stats)
        return loss.reshape(()), stats

    @staticmethod
    def backward(ctx, g_loss, _g_stats):
        (grad,) = ctx.saved_tensors
        return (grad * g_loss).to(ctx.lp_dtype), None, None, None, None, None, None, None, None, None, None, None


def fused_ppo_loss(log_prob, old_log_prob, ref_log_prob, advantages, response_mask, weights, rollout_is_weights=None, clip_low: float = 0.2,
                   clip_high: float = 0.2, clip_c: float = 3.0, kl_type: Optional[str] = None, kl_coef: float = 0.0):
    """→ (scalar loss with gradient to ``log_prob``, stats[7]): stats = [n clipped-high, Σ −(lp−old), n clipped-lower, Σ kl,
    n tokens, weighted Σ pg, weighted Σ kl] over masked tokens."""
    return _FusedPPOLoss.apply(log_prob, old_log_prob, ref_log_prob if kl_type else None, advantages, weights, response_mask, rollout_is_weights,
                               clip_low, clip_high, clip_c, KL_TYPES[kl_type], kl_coef)


def grpo_advantage(scores: torch.Tensor, group_index: torch.Tensor, response_mask: torch.Tensor, eps: float = 1e-6,
                   norm_by_std: bool = True) -> torch.Tensor:
    """``(score − mean_group) / (std_group + eps)`` broadcast over the response window (singleton groups: mean 0, std 1)."""
    if scores.is_cuda and _ext.available():
        G = int(group_index.max().item()) + 1 if group_index.numel() else 0
        return _ext.ops().grpo_advantage(scores.float().contiguous(), group_index.to(torch.int32).contiguous(), G,
                                         response_mask.float().contiguous(), float(eps), bool(norm_by_std))
    from verl_b200.utils.groupwise import group_mean_std

    mean, std, _ = group_mean_std(scores, group_index.long(), eps)
    a = scores.float() - mean[group_index.long()]
    if norm_by_std:
        a = a / (std[group_index.long()] + eps)
    return a[:, None] * response_mask.float()


def gae_advantage(token_level_rewards: torch.Tensor, values: torch.Tensor, response_mask: torch.Tensor, gamma: float, lam: float,
                  whiten: bool = True):
    """GAE over the response window in one kernel (one thread per trajectory walks backwards; masked positions carry the state
    through), optionally followed by the masked whitening of the advantages. → (advantages, returns), both fp32 [B, R]."""
    f = lambda t: t.detach().float().contiguous()          # noqa: E731
    return _ext.ops().gae(f(token_level_rewards), f(values), f(response_mask), float(gamma), float(lam), bool(whiten))


class _FusedValueLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, vpreds, values, returns, weight, mask, clip):
        f = lambda t: t.detach().float().contiguous()      # noqa: E731
        grad, stats = _ext.ops().value_loss(f(vpreds), f(values), f(returns), f(weight), f(mask), float(clip))
        ctx.save_for_backward(grad)
        ctx.v_dtype = vpreds.dtype
        ctx.mark_non_differentiable(stats)
        return stats[0].clone(), stats

    @staticmethod
    def backward(ctx, g_loss, _g_stats):
        (grad,) = ctx.saved_tensors
        return (grad * g_loss).to(ctx.v_dtype), None, None, None, None, None


def fused_value_loss(vpreds, values, returns, response_mask, weights, cliprange_value: float):
    """→ (0.5 · Σ w · max((v − R)², (clip(v, v_old ± ε) − R)²) with gradient to ``vpreds``, clipped fraction)."""
    loss, stats = _FusedValueLoss.apply(vpreds, values, returns, weights, response_mask, cliprange_value)
    return loss, stats[1] / stats[2].clamp_min(1.0)
