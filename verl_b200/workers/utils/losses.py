"""Loss adapters between engine outputs (per-token log-probs / entropy / values in the response window) and the
algorithm layer.

Parity target: ``verl/workers/utils/losses.py`` (sft_loss :28, ppo_loss :57, value_loss :158).
"""

from __future__ import annotations

from typing import Any

import torch

from verl_b200.trainer.ppo import core_algos
from verl_b200.utils import torch_functional as VF
from verl_b200.utils.metric import AggregationType, Metric

__all__ = ["ppo_loss", "value_loss", "sft_loss"]


def _get(cfg, key, default=None):
    if cfg is None:
        return default
    v = cfg.get(key, default) if hasattr(cfg, "get") else getattr(cfg, key, default)
    return default if v is None else v


class _LossCfgView(dict):
    """dict view handed to policy-loss functions: actor config + per-call global batch info."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e


def _distillation_term(distillation, model_output: dict, data, mask, agg_mode: str, info: dict):
    from verl_b200.trainer.distillation.losses import DISTILLATION_LOSSES

    if "student_topk_log_probs" not in model_output:
        raise RuntimeError("distillation is enabled but the engine produced no student_topk_log_probs: the batch needs "
                           "teacher_topk_ids / teacher_topk_log_probs (the teacher pass did not run)")
    kind = _get(distillation, "loss", "forward_kl")
    kw = {"beta": float(_get(distillation, "jsd_beta", 0.5))} if kind == "jsd" else {}
    per_tok = DISTILLATION_LOSSES[kind](model_output["student_topk_log_probs"], data["teacher_topk_log_probs"].to(mask.device), **kw)
    loss = core_algos.agg_loss(per_tok, mask, agg_mode, **info)
    with torch.no_grad():
        agree = (model_output["student_topk_log_probs"].argmax(-1) == 0).float()      # the teacher's head is sorted: index 0 is its top-1
        m = {"distill/" + kind: Metric(AggregationType.MEAN, loss.detach().item()),
             "distill/top1_agreement": Metric(AggregationType.MEAN, VF.masked_mean(agree, mask).item())}
    return loss, m


def ppo_loss(config, model_output: dict, data, dp_group=None, distillation=None) -> tuple[torch.Tensor, dict[str, Any]]:
    """Policy loss (+ entropy bonus, + KL-to-reference loss) on one micro-batch.

    ``model_output`` holds ``log_probs`` and optionally ``entropy`` as [bs, R]; ``data`` holds ``old_log_probs``,
    ``advantages``, ``response_mask`` (+ ``ref_log_prob``, ``rollout_is_weights``) and the normalisation info
    ``dp_size / batch_num_tokens / global_batch_size``.
    """
    log_prob = model_output["log_probs"]
    entropy = model_output.get("entropy")
    mask = data["response_mask"].to(log_prob.dtype)
    info = {k: data[k] for k in ("dp_size", "batch_num_tokens", "global_batch_size", "loss_scale_factor") if k in data and data[k] is not None}
    if distillation is not None and _get(distillation, "enable", False):
        # on-policy distillation: divergence to the teacher's top-k head on the student's own samples, optionally on top of
        # the policy-gradient loss (reference: verl/trainer/distillation/losses.py, distillation.loss_settings)
        d_loss, d_metrics = _distillation_term(distillation, model_output, data, mask, _get(config, "loss_agg_mode", "token-mean"), info)
        coef = float(_get(distillation, "loss_coef", 1.0))
        if not _get(distillation, "use_policy_loss", False):
            return coef * d_loss, d_metrics
        pg, m = ppo_loss(config, model_output, data, dp_group)
        m.update(d_metrics)
        return pg + coef * d_loss, m
    loss_mode = _get(_get(config, "policy_loss", {}), "loss_mode", "vanilla")
    agg_mode = _get(config, "loss_agg_mode", "token-mean")
    view = _LossCfgView({k: _get(config, k) for k in ("clip_ratio", "clip_ratio_low", "clip_ratio_high", "clip_ratio_c",
                                                       "policy_loss", "tau_pos", "tau_neg")})
    view["global_batch_info"] = info
    from verl_b200.ops import rl as rl_ops

    kl_type = _get(config, "kl_loss_type", "low_var_kl") if _get(config, "use_kl_loss", False) else None
    if loss_mode == "vanilla" and rl_ops.fused_ppo_available(log_prob) and kl_type in rl_ops.KL_TYPES and "sc_correction" not in model_output:
        # one kernel: surrogate + KL term, their gradient and the logging sums
        clip = _get(config, "clip_ratio", 0.2)
        lo, hi = _get(config, "clip_ratio_low", None), _get(config, "clip_ratio_high", None)
        w = rl_ops.agg_weights(mask, agg_mode, **info)
        coef = _get(config, "kl_loss_coef", 0.001) if kl_type else 0.0
        loss, stats = rl_ops.fused_ppo_loss(log_prob, data["old_log_probs"], data.get("ref_log_prob") if hasattr(data, "get") else None,
                                            data["advantages"], mask, w, data.get("rollout_is_weights") if hasattr(data, "get") else None,
                                            clip if lo is None else lo, clip if hi is None else hi, _get(config, "clip_ratio_c", 3.0), kl_type, coef)
        metrics = {}
        if entropy is not None and _get(config, "entropy_coeff", 0.0) != 0:
            ent_loss = core_algos.agg_loss(entropy, mask, agg_mode, **info)
            loss = loss - _get(config, "entropy_coeff", 0.0) * ent_loss
            metrics["actor/entropy_loss"] = Metric(AggregationType.MEAN, ent_loss.detach().item())
        st = stats.tolist()
        n = max(st[4], 1.0)
        metrics.update({"actor/pg_clipfrac": Metric(AggregationType.MEAN, st[0] / n), "actor/ppo_kl": Metric(AggregationType.MEAN, st[1] / n),
                        "actor/pg_clipfrac_lower": Metric(AggregationType.MEAN, st[2] / n), "actor/pg_loss": Metric(AggregationType.MEAN, st[5])})
        if kl_type:
            metrics["actor/kl_loss"] = Metric(AggregationType.MEAN, st[6])
            metrics["actor/kl_coef"] = Metric(AggregationType.MEAN, coef)
        return loss, metrics
    fn = core_algos.get_policy_loss_fn(loss_mode)
    rc = _get(_get(config, "policy_loss", {}) or {}, "rollout_correction", None) or {}
    sc_kwargs = {}
    if _get(rc, "score_centering", False):
        if "sc_correction" not in model_output:
            # a pass that never computed the head log-probs would silently train plain bypass policy gradient
            raise RuntimeError("score centering is enabled but the engine produced no sc_correction: the batch needs "
                               "rollout_topk_ids / rollout_topk_log_probs (rollout.topk_log_probs > 0)")
        sc_kwargs["sc_correction"] = model_output["sc_correction"]
    pg_loss, pg_metrics = fn(old_log_prob=data["old_log_probs"], log_prob=log_prob, advantages=data["advantages"],
                             response_mask=mask, loss_agg_mode=agg_mode, config=view,
                             rollout_is_weights=data.get("rollout_is_weights") if hasattr(data, "get") else None, **sc_kwargs)
    metrics: dict[str, Any] = {k: Metric(AggregationType.MEAN, v) for k, v in pg_metrics.items()}
    if sc_kwargs:
        for key in ("sc_sampler_head_mass", "sc_train_head_mass"):
            if key in model_output:
                metrics[f"actor/{key}"] = Metric(AggregationType.MEAN, VF.masked_mean(model_output[key].detach(), mask).item())
    loss = pg_loss
    ent_coeff = _get(config, "entropy_coeff", 0.0)
    if entropy is not None and ent_coeff != 0:
        ent_loss = core_algos.agg_loss(entropy, mask, agg_mode, **info)
        loss = loss - ent_coeff * ent_loss
        metrics["actor/entropy_loss"] = Metric(AggregationType.MEAN, ent_loss.detach().item())
    if _get(config, "use_kl_loss", False):
        kld = core_algos.kl_penalty(log_prob, data["ref_log_prob"], _get(config, "kl_loss_type", "low_var_kl"))
        kl_loss = core_algos.agg_loss(kld, mask, agg_mode, **info)
        coef = _get(config, "kl_loss_coef", 0.001)
        loss = loss + coef * kl_loss
        metrics["actor/kl_loss"] = Metric(AggregationType.MEAN, kl_loss.detach().item())
        metrics["actor/kl_coef"] = Metric(AggregationType.MEAN, coef)
    metrics["actor/pg_loss"] = Metric(AggregationType.MEAN, pg_loss.detach().item())
    return loss, metrics


def value_loss(config, model_output: dict, data, dp_group=None):
    vpreds = model_output["values"]
    mask = data["response_mask"].to(vpreds.dtype)
    info = {k: data[k] for k in ("dp_size", "batch_num_tokens", "global_batch_size") if k in data and data[k] is not None}
    from verl_b200.ops import rl as rl_ops

    if rl_ops.fused_ppo_available(vpreds):
        # one pass: clipped value loss, its gradient and the clip fraction
        w = rl_ops.agg_weights(mask, _get(config, "loss_agg_mode", "token-mean"), **info)
        loss, clipfrac = rl_ops.fused_value_loss(vpreds, data["values"], data["returns"], mask, w, _get(config, "cliprange_value", 0.5))
    else:
        loss, clipfrac = core_algos.compute_value_loss(vpreds, data["returns"], data["values"], mask,
                                                       _get(config, "cliprange_value", 0.5),
                                                       _get(config, "loss_agg_mode", "token-mean"), **info)
    metrics = {
        "critic/vf_loss": Metric(AggregationType.MEAN, loss.detach().item()),
        "critic/vf_clipfrac": Metric(AggregationType.MEAN, clipfrac.detach().item()),
        "critic/vpred_mean": Metric(AggregationType.MEAN, VF.masked_mean(vpreds, mask).detach().item()),
    }
    return loss, metrics


def sft_loss(config, model_output: dict, data, dp_group=None):
    """Negative log-likelihood over loss-masked tokens, normalised by the global token count."""
    log_prob = model_output["log_probs"]
    mask = data["loss_mask"].to(log_prob.dtype)
    n = data.get("batch_num_tokens") if hasattr(data, "get") else None
    dp = data.get("dp_size", 1) if hasattr(data, "get") else 1
    denom = n if n is not None else mask.sum().clamp(min=1)
    loss = -(log_prob * mask).sum() / denom * dp
    return loss, {"sft/loss": Metric(AggregationType.MEAN, loss.detach().item() / dp)}
