"""Rollout correction: importance-sampling weights, rejection-sampling masks and off-policy diagnostics between the
policy that generated the samples (rollout engine, possibly fp8) and the policy being trained.

Parity target: ``verl/trainer/ppo/rollout_corr_helper.py`` (rejection mask :197, IS weights :522, combined entry
point :786, off-policy metrics :904, batch helper :1013, bypass mode :1109).
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch

from verl_b200.utils import torch_functional as VF

SAFETY_BOUND = 20.0
TOKEN_LEVEL_RS = {"token_k1", "token_k2", "token_k3"}
SUPPORTED_RS = TOKEN_LEVEL_RS | {f"seq_{agg}_k{k}" for agg in ("sum", "mean") for k in (1, 2, 3)} | {"seq_max_k2", "seq_max_k3"}


def _parse_is_threshold(spec) -> tuple[float, Optional[float]]:
    """``2.0`` → (2.0, None) truncation; ``"0.5_2.0"`` → (2.0, 0.5) keep-inside-band (IcePop)."""
    if isinstance(spec, (int, float)):
        upper, lower = float(spec), None
    elif isinstance(spec, str):
        s = spec.strip()
        try:
            if "_" in s:
                lo, up = s.split("_", 1)
                lower, upper = float(lo), float(up)
            else:
                upper, lower = float(s), None
        except ValueError as exc:
            raise ValueError(f"Invalid rollout_is_threshold '{spec}'.") from exc
    else:
        raise TypeError("rollout_is_threshold must be a float or a string threshold specification.")
    if upper <= 0:
        raise ValueError(f"rollout_is_threshold upper bound must be positive, got {upper}.")
    if lower is not None and (lower <= 0 or lower > upper):
        raise ValueError("rollout_is_threshold lower bound must be positive and <= upper bound.")
    return upper, lower


def _parse_rs_thresholds(options: list[str], spec) -> dict[str, dict[str, Optional[float]]]:
    if isinstance(spec, (int, float)):
        parts = [str(spec)] * len(options)
    else:
        parts = [p.strip() for p in str(spec).split(",") if p.strip()]
        if len(parts) == 1 and len(options) > 1:
            parts = parts * len(options)
    if len(parts) != len(options):
        raise ValueError(f"rollout_rs_threshold needs one entry per rollout_rs option ({len(options)}), got {len(parts)}")
    out = {}
    for opt, p in zip(options, parts):
        if "_" in p:
            lo, up = p.split("_", 1)
            lower, upper = float(lo), float(up)
        else:
            upper = float(p)
            lower = (1.0 / upper) if opt.endswith("k1") else None
        if upper <= 0 or (lower is not None and lower <= 0):
            raise ValueError(f"thresholds must be positive, got '{p}' for {opt}")
        out[opt] = {"lower": lower, "upper": upper}
    return out


def compute_rollout_rejection_mask(log_ratio, response_mask, rollout_rs: str = "token_k1", rollout_rs_threshold=None):
    """Hard trust region: drop tokens/sequences whose divergence estimate exceeds a threshold.

    ``rollout_rs`` is a comma-separated list of criteria (all must pass): ``token_k{1,2,3}``, ``seq_sum_k{1,2,3}``,
    ``seq_mean_k{1,2,3}``, ``seq_max_k{2,3}`` where k1 = −log ρ (two-sided band given as ratio bounds ``lo_hi``),
    k2 = ½ log²ρ, k3 = ρ − 1 − log ρ.
    """
    if not rollout_rs or not isinstance(rollout_rs, str):
        raise ValueError("rollout_rs must be a non-empty string (comma separated for multiple options).")
    if rollout_rs_threshold is None:
        raise ValueError("rollout_rs_threshold must be provided for rejection sampling.")
    if log_ratio.shape[0] == 0:
        return response_mask, {}
    options = []
    for o in (x.strip() for x in rollout_rs.split(",")):
        if not o:
            continue
        if o not in SUPPORTED_RS:
            raise ValueError(f"Invalid rollout_rs option: {o}. Must be one of {sorted(SUPPORTED_RS)}.")
        if o not in options:
            options.append(o)
    if not options:
        raise ValueError("rollout_rs must contain at least one valid option.")
    th = _parse_rs_thresholds(options, rollout_rs_threshold)
    lr = torch.clamp(log_ratio, min=-SAFETY_BOUND, max=SAFETY_BOUND)
    stats = {"k1": -lr, "k2": 0.5 * lr**2, "k3": torch.exp(lr) - 1.0 - lr}
    mask_b = response_mask.bool()
    seq_valid = response_mask.sum(dim=-1) > 0
    keep_all = torch.ones_like(response_mask, dtype=log_ratio.dtype)
    metrics: dict[str, float] = {}
    for opt in options:
        k = opt[-2:]
        tok = stats[k]
        up, lo = th[opt]["upper"], th[opt]["lower"]
        if opt in TOKEN_LEVEL_RS:
            stat = tok
        else:
            agg = opt.split("_")[1]
            if agg == "sum":
                seq = VF.masked_sum(tok, response_mask, axis=-1)
            elif agg == "mean":
                seq = VF.masked_mean(tok, response_mask, axis=-1)
            else:
                seq = tok.masked_fill(~mask_b, float("-inf")).max(dim=-1).values
                seq = torch.where(torch.isinf(seq), torch.zeros_like(seq), seq)
            stat = seq.unsqueeze(-1).expand_as(response_mask)
        if k == "k1":
            keep = (stat >= math.log(lo)) & (stat <= math.log(up))
        else:
            keep = stat <= up
        keep_f = keep.to(log_ratio.dtype)
        keep_all = keep_all * keep_f
        seq_keep = (~((~keep) & mask_b)).all(dim=-1)
        metrics[f"rollout_rs_{opt}_mean"] = VF.masked_mean(stat, response_mask).item()
        metrics[f"rollout_rs_{opt}_max"] = stat.masked_fill(~mask_b, float("-inf")).max().item()
        metrics[f"rollout_rs_{opt}_masked_fraction"] = VF.masked_mean(1 - keep_f, response_mask).item()
        sv = seq_valid.float()
        metrics[f"rollout_rs_{opt}_seq_masked_fraction"] = (
            (((1.0 - seq_keep.to(log_ratio.dtype)) * sv).sum() / sv.sum()).item() if sv.sum() > 0 else 0.0
        )
    new_mask = response_mask * keep_all.to(response_mask.dtype)
    metrics["rollout_rs_masked_fraction"] = VF.masked_mean(1 - keep_all, response_mask).item()
    return new_mask, metrics


def compute_rollout_correction_weights(log_ratio, response_mask, rollout_is: str = "token", rollout_is_threshold=2.0,
                                       rollout_is_batch_normalize: bool = False):
    """Truncated importance weights ρ = π_train/π_rollout at token or sequence level (detached)."""
    if rollout_is not in ("token", "sequence"):
        raise ValueError(f"Invalid rollout_is: {rollout_is}. Must be one of {{'token', 'sequence'}}.")
    upper, lower = _parse_is_threshold(rollout_is_threshold)
    if rollout_is == "token":
        lr_metric = log_ratio
        raw = torch.exp(torch.clamp(log_ratio, min=-SAFETY_BOUND, max=SAFETY_BOUND))
    else:
        lr_metric = VF.masked_sum(log_ratio, response_mask, axis=-1).unsqueeze(-1)
        raw = torch.exp(torch.clamp(lr_metric, min=-SAFETY_BOUND, max=SAFETY_BOUND)).expand_as(log_ratio)
    raw = raw * response_mask
    if lower is None:
        w = raw.clamp(max=upper)
    else:
        w = torch.where((raw >= lower) & (raw <= upper), raw, torch.zeros_like(raw))
    metrics = compute_is_metrics(w, raw, lr_metric, response_mask, rollout_is, upper, lower)
    if lower is not None:
        metrics["rollout_is_oob_ratio"] = VF.masked_mean(((raw < lower) | (raw > upper)).float(), response_mask).item()
    w = w.detach()
    if rollout_is_batch_normalize:
        dist_on = torch.distributed.is_available() and torch.distributed.is_initialized()
        if rollout_is == "token":
            mean = VF.distributed_masked_mean(w, response_mask.to(w.dtype)) if dist_on else VF.masked_mean(w, response_mask)
        else:
            sw = VF.masked_mean(w, response_mask, axis=-1)
            sm = (response_mask.sum(dim=-1) > 0).to(w.dtype)
            mean = VF.distributed_masked_mean(sw, sm) if dist_on else (sw * sm).sum() / sm.sum().clamp_min(1e-8)
        if mean > 1e-8:
            w = w / mean
            metrics["rollout_is_batch_norm_factor"] = float(mean)
        else:
            metrics["rollout_is_batch_norm_factor"] = 1.0
    return w, metrics


def compute_is_metrics(weights, raw_weights, log_ratio_for_metrics, response_mask, rollout_is, upper, lower=None) -> dict:
    m: dict[str, float] = {}
    mask_b = response_mask.bool()
    m["rollout_is_mean"] = VF.masked_mean(weights, response_mask).item()
    valid = weights[mask_b] if mask_b.any() else weights.new_zeros(1)
    m["rollout_is_max"] = valid.max().item()
    m["rollout_is_min"] = valid.min().item()
    m["rollout_is_std"] = valid.std().item() if valid.numel() > 1 else 0.0
    mean_w = valid.mean().clamp_min(1e-12)
    m["rollout_is_eff_sample_size"] = (1.0 / ((valid / mean_w) ** 2).mean().clamp_min(1e-12)).item()
    log_up = math.log(upper)
    if rollout_is == "sequence":
        lr_seq = log_ratio_for_metrics.squeeze(-1)
        m["rollout_is_ratio_fraction_high"] = (lr_seq > log_up).float().mean().item()
        if lower is not None:
            m["rollout_is_ratio_fraction_low"] = (lr_seq < math.log(lower)).float().mean().item()
        sw = torch.exp(torch.clamp(lr_seq, -SAFETY_BOUND, SAFETY_BOUND))
        m["rollout_is_seq_mean"], m["rollout_is_seq_max"], m["rollout_is_seq_min"] = sw.mean().item(), sw.max().item(), sw.min().item()
    else:
        m["rollout_is_ratio_fraction_high"] = VF.masked_mean((log_ratio_for_metrics > log_up).float(), response_mask).item()
        if lower is not None:
            m["rollout_is_ratio_fraction_low"] = VF.masked_mean((log_ratio_for_metrics < math.log(lower)).float(), response_mask).item()
    return m


def compute_offpolicy_metrics(old_log_prob, rollout_log_prob, response_mask) -> dict[str, Any]:
    """KL / perplexity / χ² diagnostics of the gap between the training policy and the rollout policy."""
    assert response_mask.any(), "Expected at least one valid token in response_mask"
    m = {}
    mlp_train = VF.masked_mean(old_log_prob, response_mask, axis=-1)
    m["training_ppl"] = torch.exp(-mlp_train).mean().item()
    m["training_log_ppl"] = (-mlp_train).mean().item()
    if rollout_log_prob is not None:
        m["kl"] = VF.masked_mean(rollout_log_prob - old_log_prob, response_mask).item()
        lr = old_log_prob - rollout_log_prob
        m["k3_kl"] = VF.masked_mean(torch.exp(lr) - lr - 1, response_mask).item()
        mlp_roll = VF.masked_mean(rollout_log_prob, response_mask, axis=-1)
        m["rollout_ppl"] = torch.exp(-mlp_roll).mean().item()
        m["rollout_log_ppl"] = (-mlp_roll).mean().item()
        d = mlp_roll - mlp_train
        m["log_ppl_diff"], m["log_ppl_abs_diff"] = d.mean().item(), d.abs().mean().item()
        m["log_ppl_diff_max"], m["log_ppl_diff_min"] = d.max().item(), d.min().item()
        m["ppl_ratio"] = torch.exp(d).mean().item()
        rho = torch.exp(torch.clamp(lr, -SAFETY_BOUND, SAFETY_BOUND))
        m["chi2_token"] = (VF.masked_mean(rho.square(), response_mask) - 1.0).item()
        lrs = torch.clamp(VF.masked_sum(lr, response_mask, axis=-1), -SAFETY_BOUND, SAFETY_BOUND)
        m["chi2_seq"] = (torch.exp(2.0 * lrs).mean() - 1.0).item()
    return m


def compute_rollout_correction_and_rejection_mask(old_log_prob, rollout_log_prob, response_mask, rollout_is=None,
                                                  rollout_is_threshold=2.0, rollout_rs=None, rollout_rs_threshold=None,
                                                  rollout_is_batch_normalize=False):
    """Returns (is_weights or None, possibly-modified response_mask, metrics prefixed ``rollout_corr/``)."""
    log_ratio = old_log_prob - rollout_log_prob
    metrics: dict[str, float] = {}
    weights = None
    if rollout_is is not None:
        weights, m = compute_rollout_correction_weights(log_ratio, response_mask, rollout_is, rollout_is_threshold,
                                                        rollout_is_batch_normalize)
        metrics.update(m)
    mask = response_mask
    if rollout_rs is not None:
        mask, m = compute_rollout_rejection_mask(log_ratio, response_mask, rollout_rs, rollout_rs_threshold)
        metrics.update(m)
    metrics.update(compute_offpolicy_metrics(old_log_prob, rollout_log_prob, response_mask))
    return weights, mask, {f"rollout_corr/{k}": (v.item() if torch.is_tensor(v) else v) for k, v in metrics.items()}


def compute_rollout_correction_and_add_to_batch(batch, rollout_corr_config):
    """Trainer-side entry: adds ``rollout_is_weights`` and replaces ``response_mask`` in the DataProto."""
    g = (lambda k, d=None: rollout_corr_config.get(k, d)) if hasattr(rollout_corr_config, "get") else (lambda k, d=None: getattr(rollout_corr_config, k, d))
    w, mask, metrics = compute_rollout_correction_and_rejection_mask(
        batch.batch["old_log_probs"], batch.batch["rollout_log_probs"], batch.batch["response_mask"],
        rollout_is=g("rollout_is"), rollout_is_threshold=g("rollout_is_threshold", 2.0), rollout_rs=g("rollout_rs"),
        rollout_rs_threshold=g("rollout_rs_threshold"), rollout_is_batch_normalize=g("rollout_is_batch_normalize", False))
    if w is not None:
        batch.batch["rollout_is_weights"] = w
    batch.batch["response_mask"] = mask
    return batch, metrics


def compute_rollout_corr_metrics_from_logprobs(log_prob, rollout_log_prob, response_mask) -> dict:
    m = compute_offpolicy_metrics(log_prob, rollout_log_prob, response_mask)
    return {f"rollout_corr/{k}": v for k, v in m.items()}


def apply_bypass_mode(batch, rollout_corr_config, policy_loss_config: dict):
    """Use the rollout log-probs as ``old_log_probs`` (skips the recompute pass) and route the actor to the
    ``bypass_mode`` loss, which applies IS/RS corrections itself."""
    if "rollout_log_probs" not in batch.batch:
        raise ValueError("bypass_mode=True requires rollout_log_probs in batch (rollout.calculate_log_probs=true).")
    batch.batch["old_log_probs"] = batch.batch["rollout_log_probs"]
    policy_loss_config["rollout_correction"] = rollout_corr_config
    policy_loss_config["loss_mode"] = "bypass_mode"
    return batch
