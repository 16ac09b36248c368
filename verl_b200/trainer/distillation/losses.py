"""On-policy distillation losses between the student's distribution and a teacher's top-k head
(reference: ``verl/trainer/distillation/losses.py`` and the fsdp / megatron variants).

Inputs are per-token: ``student_logp [T, k]`` — the student's full-vocabulary-normalised log-probs at the teacher's top-k
ids (see ``trainer.ppo.score_centering.topk_log_probs_from_hidden`` for a logits-free way to get them) — and
``teacher_logp [T, k]``. The probability mass outside the head is folded into one extra "tail" bucket on both sides so
every divergence is taken between proper (k+1)-point distributions.
"""

from __future__ import annotations

import math

import torch

__all__ = ["with_tail_bucket", "forward_kl", "reverse_kl", "jsd", "topk_distillation_loss", "DISTILLATION_LOSSES"]


def with_tail_bucket(logp: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    """[T, k] head log-probs → [T, k+1] with ``log(1 − Σ head)`` appended."""
    mass = logp.float().exp().sum(-1, keepdim=True).clamp(max=1.0 - eps)
    return torch.cat([logp.float(), torch.log1p(-mass).clamp_min(math.log(eps))], -1)


def forward_kl(student_logp: torch.Tensor, teacher_logp: torch.Tensor) -> torch.Tensor:
    """KL(teacher ‖ student): mass-covering."""
    s, t = with_tail_bucket(student_logp), with_tail_bucket(teacher_logp)
    return (t.exp() * (t - s)).sum(-1)


def reverse_kl(student_logp: torch.Tensor, teacher_logp: torch.Tensor) -> torch.Tensor:
    """KL(student ‖ teacher): mode-seeking."""
    s, t = with_tail_bucket(student_logp), with_tail_bucket(teacher_logp)
    return (s.exp() * (s - t)).sum(-1)


def jsd(student_logp: torch.Tensor, teacher_logp: torch.Tensor, beta: float = 0.5) -> torch.Tensor:
    """Generalised Jensen–Shannon divergence with mixture ``m = β·teacher + (1−β)·student``."""
    s, t = with_tail_bucket(student_logp), with_tail_bucket(teacher_logp)
    m = torch.logaddexp(t + math.log(beta), s + math.log(1 - beta))
    return beta * (t.exp() * (t - m)).sum(-1) + (1 - beta) * (s.exp() * (s - m)).sum(-1)


DISTILLATION_LOSSES = {"forward_kl": forward_kl, "reverse_kl": reverse_kl, "jsd": jsd}


def topk_distillation_loss(student_logp: torch.Tensor, teacher_logp: torch.Tensor, loss_mask: torch.Tensor, kind: str = "forward_kl",
                           loss_agg_mode: str = "token-mean", **kwargs):
    """Masked aggregate of the chosen divergence; returns (loss, metrics)."""
    from verl_b200.trainer.ppo.core_algos import agg_loss

    per_tok = DISTILLATION_LOSSES[kind](student_logp, teacher_logp, **kwargs)
    shape = loss_mask.shape
    loss = agg_loss(per_tok.reshape(shape), loss_mask.float(), loss_agg_mode)
    with torch.no_grad():
        agree = (student_logp.argmax(-1) == teacher_logp.argmax(-1)).float().reshape(shape)
        m = loss_mask.float()
        metrics = {f"distill/{kind}": float(loss.detach()), "distill/top1_agreement": float((agree * m).sum() / m.sum().clamp_min(1)),
                   "distill/teacher_head_mass": float((teacher_logp.float().exp().sum(-1).reshape(shape) * m).sum() / m.sum().clamp_min(1))}
    return loss, metrics
