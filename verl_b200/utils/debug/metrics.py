"""Agreement between the rollout engine's log-probs and the trainer's recomputed ones
(reference: ``verl/utils/debug/metrics.py:23-110``)."""

import torch

from verl_b200.protocol import DataProto


def calculate_token_list_diff(a: torch.Tensor, b: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return torch.where(mask.bool(), (a - b).abs(), torch.zeros_like(a))


def pearson_correlation_coefficient(x: torch.Tensor, y: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    x, y = torch.masked_select(x, mask.bool()), torch.masked_select(y, mask.bool())
    if x.numel() < 2:
        return torch.tensor(0.0)
    xm, ym = x - x.mean(), y - y.mean()
    return (xm * ym).sum() / (xm.norm() * ym.norm() + 1e-12)


def calculate_debug_metrics(data: DataProto) -> dict:
    rollout_lp = data.batch["rollout_log_probs"]
    actor_lp = data.batch["old_log_probs"]
    mask = data.batch["response_mask"] if "response_mask" in data.batch.keys() else data.batch["attention_mask"][:, -rollout_lp.shape[1]:]
    rp, ap = torch.exp(rollout_lp), torch.exp(actor_lp)
    diff = torch.masked_select(calculate_token_list_diff(rp, ap, mask), mask.bool())
    if diff.numel() == 0:
        return {}
    return {"training/rollout_probs_diff_max": diff.max().item(), "training/rollout_probs_diff_mean": diff.mean().item(),
            "training/rollout_probs_diff_std": diff.std().item() if diff.numel() > 1 else 0.0,
            "training/rollout_actor_probs_pearson_corr": pearson_correlation_coefficient(rp, ap, mask).item()}
