"""RL algorithm core: advantage estimators, policy losses, KL penalties, loss aggregation, value loss.

Everything here is pure tensor math that runs identically on CPU (oracle) and GPU. Group statistics are computed
with segment reductions over integer group ids (no per-sample Python loops), so the GRPO/RLOO family stays
launch-light at 2048 samples per step.

Parity target: ``verl/trainer/ppo/core_algos.py`` — registries (:53, :116), KL controllers (:153-212),
estimators (:215-1121), ``agg_loss`` (:1140), policy losses (:1285-2105, :2333-2559), value loss (:2125),
``kl_penalty`` (:2188-2251), PF-PPO resampling (:2254).
"""

from __future__ import annotations

from enum import Enum
from typing import Any, Callable, Optional

import numpy as np
import torch

from verl_b200.utils import torch_functional as VF

__all__ = [
    "register_adv_est", "get_adv_estimator_fn", "AdvantageEstimator", "register_policy_loss", "get_policy_loss_fn",
    "AdaptiveKLController", "FixedKLController", "get_kl_controller", "agg_loss", "compute_policy_loss",
    "compute_value_loss", "compute_entropy_loss", "kl_penalty", "kl_penalty_forward", "compute_rewards",
    "compute_pf_ppo_reweight_data", "group_ids_from_index",
]

POLICY_LOSS_REGISTRY: dict[str, Callable] = {}
ADV_ESTIMATOR_REGISTRY: dict[str, Callable] = {}


def register_policy_loss(name: str):
    def deco(fn):
        POLICY_LOSS_REGISTRY[name] = fn
        return fn

    return deco


def get_policy_loss_fn(name: str):
    if name not in POLICY_LOSS_REGISTRY:
        raise ValueError(f"Unsupported loss mode: {name}. Supported modes are: {sorted(POLICY_LOSS_REGISTRY)}")
    return POLICY_LOSS_REGISTRY[name]


class AdvantageEstimator(str, Enum):
    GAE = "gae"
    GRPO = "grpo"
    GRPO_VECTORIZED = "grpo_vectorized"
    GDPO = "gdpo"
    REINFORCE_PLUS_PLUS = "reinforce_plus_plus"
    REINFORCE_PLUS_PLUS_BASELINE = "reinforce_plus_plus_baseline"
    REMAX = "remax"
    RLOO = "rloo"
    OPO = "opo"
    GRPO_PASSK = "grpo_passk"
    GPG = "gpg"
    RLOO_VECTORIZED = "rloo_vectorized"
    OPTIMAL_TOKEN_BASELINE = "optimal_token_baseline"
    TIR_OPTIMAL_TOKEN_BASELINE = "tir_optimal_token_baseline"


def register_adv_est(name_or_enum):
    def deco(fn):
        name = name_or_enum.value if isinstance(name_or_enum, Enum) else name_or_enum
        if name in ADV_ESTIMATOR_REGISTRY and ADV_ESTIMATOR_REGISTRY[name] is not fn:
            raise ValueError(f"Adv estimator {name} has already been registered")
        ADV_ESTIMATOR_REGISTRY[name] = fn
        return fn

    return deco


def get_adv_estimator_fn(name_or_enum):
    name = name_or_enum.value if isinstance(name_or_enum, Enum) else name_or_enum
    if name not in ADV_ESTIMATOR_REGISTRY:
        raise ValueError(f"Unknown advantage estimator: {name}")
    return ADV_ESTIMATOR_REGISTRY[name]


# ------------------------------------------------------------------------------------------------ KL control
class AdaptiveKLController:
    """Proportional controller on the KL coefficient (Ziegler et al. 2019)."""

    def __init__(self, init_kl_coef: float, target_kl: float, horizon: int):
        self.value = init_kl_coef
        self.target = target_kl
        self.horizon = horizon

    def update(self, current_kl: float, n_steps: int):
        err = float(np.clip(current_kl / self.target - 1, -0.2, 0.2))
        self.value *= 1 + err * n_steps / self.horizon


class FixedKLController:
    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current_kl: float, n_steps: int):
        pass


def get_kl_controller(kl_ctrl):
    t = kl_ctrl.get("type", "fixed") if hasattr(kl_ctrl, "get") else kl_ctrl.type
    g = (lambda k, d=None: kl_ctrl.get(k, d)) if hasattr(kl_ctrl, "get") else (lambda k, d=None: getattr(kl_ctrl, k, d))
    if t == "fixed":
        return FixedKLController(kl_coef=g("kl_coef"))
    if t == "adaptive":
        assert g("horizon") > 0, f"horizon must be larger than 0. Got {g('horizon')}"
        return AdaptiveKLController(init_kl_coef=g("kl_coef"), target_kl=g("target_kl"), horizon=g("horizon"))
    raise NotImplementedError(f"unknown kl controller type {t}")


# ------------------------------------------------------------------------------------------------ group helpers
def group_ids_from_index(index, device=None) -> tuple[torch.Tensor, int]:
    """Map arbitrary hashable group labels (uids) to dense int64 ids; returns (ids, num_groups)."""
    if isinstance(index, torch.Tensor):
        uniq, inv = torch.unique(index, return_inverse=True)
        return inv.to(device or index.device), int(uniq.numel())
    arr = np.asarray(index)
    _, inv = np.unique(arr.astype(str) if arr.dtype == object else arr, return_inverse=True)
    n = int(inv.max()) + 1 if inv.size else 0
    return torch.as_tensor(inv, dtype=torch.int64, device=device), n


def _group_stats(scores: torch.Tensor, gid: torch.Tensor, G: int):
    """Per-group count, mean and unbiased std of a 1-D score vector."""
    ones = torch.ones_like(scores)
    cnt = torch.zeros(G, dtype=scores.dtype, device=scores.device).index_add_(0, gid, ones)
    s1 = torch.zeros(G, dtype=scores.dtype, device=scores.device).index_add_(0, gid, scores)
    mean = s1 / cnt.clamp(min=1)
    dev2 = (scores - mean[gid]) ** 2
    s2 = torch.zeros(G, dtype=scores.dtype, device=scores.device).index_add_(0, gid, dev2)
    std = torch.sqrt(s2 / (cnt - 1).clamp(min=1))
    return cnt, mean, std


# ------------------------------------------------------------------------------------------------ estimators
@register_adv_est(AdvantageEstimator.GAE)
def compute_gae_advantage_return(token_level_rewards, values, response_mask, gamma, lam, **kwargs):
    """GAE with masked positions skipped (state carried through non-response tokens), then whitened."""
    if token_level_rewards.is_cuda:
        from verl_b200.ops import _ext

        if _ext.available():       # one scan kernel + one whitening kernel instead of a Python loop over the response length
            from verl_b200.ops.rl import gae_advantage

            if float(response_mask.sum()) < 2:
                raise ValueError("masked_var with fewer than two elements and unbiased=True")
            return gae_advantage(token_level_rewards, values, response_mask, gamma, lam, whiten=True)
    with torch.no_grad():
        nextvalues = torch.zeros_like(values[:, 0])
        lastgaelam = torch.zeros_like(values[:, 0])
        adv_rev = []
        T = token_level_rewards.shape[-1]
        for t in reversed(range(T)):
            delta = token_level_rewards[:, t] + gamma * nextvalues - values[:, t]
            cand = delta + gamma * lam * lastgaelam
            m = response_mask[:, t]
            nextvalues = values[:, t] * m + (1 - m) * nextvalues
            lastgaelam = cand * m + (1 - m) * lastgaelam
            adv_rev.append(lastgaelam)
        advantages = torch.stack(adv_rev[::-1], dim=1)
        returns = advantages + values
        advantages = VF.masked_whiten(advantages, response_mask)
    return advantages, returns


@register_adv_est(AdvantageEstimator.GRPO)
def compute_grpo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                   norm_adv_by_std_in_grpo: bool = True, config=None, **kwargs):
    """Outcome reward normalised inside each prompt group: (s − mean_g) / (std_g + ε); singleton groups → (s − 0)/1."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = group_ids_from_index(index, scores.device)
        cnt, mean, std = _group_stats(scores, gid, G)
        single = cnt <= 1
        mean = torch.where(single, torch.zeros_like(mean), mean)
        std = torch.where(single, torch.ones_like(std), std)
        if norm_adv_by_std_in_grpo:
            adv = (scores - mean[gid]) / (std[gid] + epsilon)
        else:
            adv = scores - mean[gid]
        adv = adv.unsqueeze(-1) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.GRPO_VECTORIZED)
def compute_grpo_vectorized_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                              norm_adv_by_std_in_grpo: bool = True, config=None, **kwargs):
    return compute_grpo_outcome_advantage(token_level_rewards, response_mask, index, epsilon, norm_adv_by_std_in_grpo, config)


@register_adv_est(AdvantageEstimator.GDPO)
def compute_gdpo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                   norm_adv_by_std_in_grpo: bool = True, config=None, non_tensor_batch=None,
                                   batch=None, **kwargs):
    """Normalise every reward component inside its group separately, sum with weights, whiten over the batch."""
    comps, weights = None, None
    if config is not None and non_tensor_batch is not None and batch is not None:
        keys = config.get("gdpo_reward_keys", None)
        assert keys, "GDPO requires 'algorithm.gdpo_reward_keys' naming the reward components returned by compute_score"
        dev = token_level_rewards.device
        prompt_len = batch["prompts"].size(1)
        last = batch["attention_mask"][:, prompt_len:].sum(dim=1) - 1
        comps = []
        rows = torch.arange(response_mask.size(0), device=dev)
        for k in keys:
            assert k in non_tensor_batch, f"GDPO reward key '{k}' missing from non_tensor_batch ({list(non_tensor_batch)})"
            v = torch.tensor(np.asarray(non_tensor_batch[k], dtype=np.float32), device=dev)
            m = torch.zeros_like(response_mask, dtype=torch.float32)
            m[rows, last] = v
            comps.append(m)
        w = config.get("gdpo_reward_weights", None)
        weights = list(w) if w is not None else None
    if comps is None:
        comps = [token_level_rewards]
    wt = torch.tensor(weights if weights is not None else [1.0] * len(comps), dtype=torch.float32, device=token_level_rewards.device)
    total = None
    for i, c in enumerate(comps):
        a, _ = compute_grpo_outcome_advantage(c, response_mask, index, epsilon, norm_adv_by_std_in_grpo, config)
        total = wt[i] * a if total is None else total + wt[i] * a
    adv = VF.masked_whiten(total, response_mask) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.GRPO_PASSK)
def compute_grpo_passk_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                         norm_adv_by_std_in_grpo: bool = True, config=None, **kwargs):
    """Pass@k: only the best sample of a group gets advantage r_max − r_second (optionally / std)."""
    if config is not None:
        norm_adv_by_std_in_grpo = config.get("norm_adv_by_std_in_grpo", norm_adv_by_std_in_grpo)
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = group_ids_from_index(index, scores.device)
        cnt, _, std = _group_stats(scores, gid, G)
        if bool((cnt < 2).any()):
            raise ValueError("Pass@k requires at least 2 samples per group")
        adv = torch.zeros_like(scores)
        for g in range(G):
            members = torch.nonzero(gid == g).flatten()
            top, ti = torch.topk(scores[members], 2)
            a = top[0] - top[1]
            if norm_adv_by_std_in_grpo:
                a = a / (std[g] + epsilon)
            adv[members[ti[0]]] = a
        adv = adv.unsqueeze(-1) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.REINFORCE_PLUS_PLUS_BASELINE)
def compute_reinforce_plus_plus_baseline_outcome_advantage(token_level_rewards, response_mask, index, epsilon=1e-6,
                                                           config=None, **kwargs):
    """Group-mean baseline, then batch-level whitening."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = group_ids_from_index(index, scores.device)
        cnt, mean, _ = _group_stats(scores, gid, G)
        mean = torch.where(cnt <= 1, torch.zeros_like(mean), mean)
        adv = (scores - mean[gid]).unsqueeze(-1).expand_as(response_mask) * response_mask
        adv = VF.masked_whiten(adv, response_mask) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.RLOO)
def compute_rloo_outcome_advantage(token_level_rewards, response_mask, index, epsilon=1e-6, config=None, **kwargs):
    """Leave-one-out baseline: n/(n−1)·(s − mean_g)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = group_ids_from_index(index, scores.device)
        cnt, mean, _ = _group_stats(scores, gid, G)
        n = cnt[gid]
        adv = torch.where(n > 1, (scores - mean[gid]) * n / (n - 1).clamp(min=1), scores)
        adv = adv.unsqueeze(-1) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.RLOO_VECTORIZED)
def compute_rloo_vectorized_outcome_advantage(token_level_rewards, response_mask, index, epsilon=1e-6, config=None, **kwargs):
    return compute_rloo_outcome_advantage(token_level_rewards, response_mask, index, epsilon, config)


@register_adv_est(AdvantageEstimator.OPO)
def compute_opo_outcome_advantage(token_level_rewards, response_mask, index, epsilon=1e-6, config=None, **kwargs):
    """Length-weighted group baseline: b_g = Σ len·s / Σ len."""
    with torch.no_grad():
        lens = response_mask.sum(dim=-1).to(token_level_rewards.dtype)
        scores = token_level_rewards.sum(dim=-1)
        gid, G = group_ids_from_index(index, scores.device)
        z = lambda: torch.zeros(G, dtype=scores.dtype, device=scores.device)
        cnt = z().index_add_(0, gid, torch.ones_like(scores))
        num = z().index_add_(0, gid, lens * scores)
        den = z().index_add_(0, gid, lens)
        base = torch.where(cnt > 1, num / den.clamp(min=1e-12), torch.zeros_like(num))
        adv = (scores - base[gid]).unsqueeze(-1) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.REINFORCE_PLUS_PLUS)
def compute_reinforce_plus_plus_outcome_advantage(token_level_rewards, response_mask, config=None, gamma=None, **kwargs):
    """Discounted reward-to-go (reset at masked positions), whitened over the batch."""
    if gamma is None:
        assert config is not None
        gamma = config.gamma
    with torch.no_grad():
        returns = torch.zeros_like(token_level_rewards)
        running = torch.zeros_like(token_level_rewards[:, 0])
        for t in reversed(range(token_level_rewards.shape[1])):
            running = token_level_rewards[:, t] + gamma * running
            returns[:, t] = running
            running = running * response_mask[:, t]
        adv = VF.masked_whiten(returns, response_mask) * response_mask
    return adv, returns


@register_adv_est(AdvantageEstimator.REMAX)
def compute_remax_outcome_advantage(token_level_rewards, reward_baselines, response_mask, config=None, **kwargs):
    """Reward-to-go minus the greedy-rollout baseline."""
    with torch.no_grad():
        returns = (token_level_rewards * response_mask).flip(dims=[-1]).cumsum(dim=-1).flip(dims=[-1])
        adv = returns - reward_baselines.unsqueeze(-1) * response_mask
    return adv, returns


@register_adv_est(AdvantageEstimator.GPG)
def compute_gpg_outcome_advantage(token_level_rewards, response_mask, index, epsilon=1e-6, f_norm=1.0, alpha=1.0,
                                  config=None, **kwargs):
    """GPG: α·(s − mean_g)/f_norm with α = batch / #non-zero scores."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        gid, G = group_ids_from_index(index, scores.device)
        cnt, mean, _ = _group_stats(scores, gid, G)
        mean = torch.where(cnt <= 1, torch.zeros_like(mean), mean)
        a = scores.shape[0] / torch.count_nonzero(scores).clamp(min=1)
        adv = (a * (scores - mean[gid]) / f_norm).unsqueeze(-1) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.OPTIMAL_TOKEN_BASELINE)
def compute_optimal_token_baseline_advantage(token_level_rewards, response_mask, index, old_log_probs, sum_pi_squared,
                                             rollout_is_weights=None, handle_zero_tail=False, epsilon=1e-8, config=None,
                                             **kwargs):
    """Per-timestep variance-optimal baseline B_t = Σ_g G_t·W_t / Σ_g W_t with W_t = Σ_{j≤t}(1 − 2π_j + Σπ²)."""
    with torch.no_grad():
        returns = (token_level_rewards * response_mask).flip(dims=[-1]).cumsum(dim=-1).flip(dims=[-1])
        w = 1 - 2 * torch.exp(old_log_probs) + sum_pi_squared
        if rollout_is_weights is not None:
            w = w * rollout_is_weights**2
        W = (w * response_mask).cumsum(dim=-1)
        gid, G = group_ids_from_index(index, returns.device)
        L = returns.shape[1]
        num = torch.zeros(G, L, dtype=returns.dtype, device=returns.device).index_add_(0, gid, returns * W * response_mask)
        den = torch.zeros(G, L, dtype=returns.dtype, device=returns.device).index_add_(0, gid, W * response_mask) + epsilon
        cnt = torch.zeros(G, dtype=returns.dtype, device=returns.device).index_add_(0, gid, torch.ones_like(returns[:, 0]))
        base = (num / den)[gid] * (cnt[gid] > 1).unsqueeze(-1)
        if handle_zero_tail:
            lens = response_mask.sum(-1)
            for g in range(G):
                members = torch.nonzero(gid == g).flatten()
                if members.numel() < 2:
                    continue
                sl, order = torch.sort(lens[members])
                if sl[-1] > sl[-2]:
                    base[members[order[-1]], int(sl[-2]):] = 0.0
        adv = (returns - base) * response_mask
    return adv, returns


@register_adv_est(AdvantageEstimator.TIR_OPTIMAL_TOKEN_BASELINE)
def compute_multi_turn_optimal_token_baseline_advantage(token_level_rewards, response_mask, index, old_log_probs,
                                                        sum_pi_squared, rollout_is_weights=None, handle_zero_tail=True,
                                                        epsilon=1e-8, config=None, **kwargs):
    """Tool-integrated variant: one baseline per *turn boundary*; positions inside a masked (tool) span inherit the
    cumulative variance proxy of the last model token, so tool tokens neither add variance nor get advantages."""
    with torch.no_grad():
        returns = (token_level_rewards * response_mask).flip(dims=[-1]).cumsum(dim=-1).flip(dims=[-1])
        w = (1 - 2 * torch.exp(old_log_probs) + sum_pi_squared) * response_mask
        if rollout_is_weights is not None:
            w = w * rollout_is_weights**2
        W = w.cumsum(dim=-1)
        gid, G = group_ids_from_index(index, returns.device)
        # align by model-token ordinal rather than absolute position so turns of different tool lengths line up
        ordinal = (response_mask.cumsum(-1) - 1).clamp(min=0).long()
        L = returns.shape[1]
        flat_g = gid.unsqueeze(-1).expand_as(ordinal)
        num = torch.zeros(G, L, dtype=returns.dtype, device=returns.device)
        den = torch.zeros(G, L, dtype=returns.dtype, device=returns.device)
        num.index_put_((flat_g, ordinal), returns * W * response_mask, accumulate=True)
        den.index_put_((flat_g, ordinal), W * response_mask, accumulate=True)
        cnt = torch.zeros(G, dtype=returns.dtype, device=returns.device).index_add_(0, gid, torch.ones_like(returns[:, 0]))
        base = (num / (den + epsilon))[flat_g, ordinal] * (cnt[gid] > 1).unsqueeze(-1)
        if handle_zero_tail:
            n_tok = response_mask.sum(-1)
            for g in range(G):
                members = torch.nonzero(gid == g).flatten()
                if members.numel() < 2:
                    continue
                sl, order = torch.sort(n_tok[members])
                if sl[-1] > sl[-2]:
                    row = members[order[-1]]
                    base[row] = torch.where(ordinal[row] >= int(sl[-2]), torch.zeros_like(base[row]), base[row])
        adv = (returns - base) * response_mask
    return adv, returns


def compute_rewards(token_level_scores, old_log_prob, ref_log_prob, kl_ratio):
    return token_level_scores - (old_log_prob - ref_log_prob) * kl_ratio


# ------------------------------------------------------------------------------------------------ aggregation
def agg_loss(loss_mat: torch.Tensor, loss_mask: torch.Tensor, loss_agg_mode: str, dp_size: int = 1,
             batch_num_tokens: Optional[int] = None, global_batch_size: Optional[int] = None,
             loss_scale_factor: Optional[int] = None) -> torch.Tensor:
    """Reduce a [bs, L] loss matrix to a scalar.

    The ``dp_size`` factor cancels the gradient averaging data-parallel training applies, so that summing micro-batch
    losses normalised by *global* token/sequence counts yields the exact global mean irrespective of how the
    batch was split.
    """
    if loss_agg_mode == "token-mean":
        if batch_num_tokens is None:
            if dp_size > 1:
                raise ValueError("(global) batch_num_tokens is required when dp_size > 1")
            batch_num_tokens = loss_mask.sum()
        return VF.masked_sum(loss_mat, loss_mask) / batch_num_tokens * dp_size
    if loss_agg_mode == "token-sum":
        return VF.masked_sum(loss_mat, loss_mask) * dp_size
    if loss_agg_mode in ("seq-mean-token-sum", "seq-mean-token-sum-norm"):
        seq = torch.sum(loss_mat * loss_mask, dim=-1)
        alive = (torch.sum(loss_mask, dim=-1) > 0).float()
        if global_batch_size is None:
            if dp_size > 1:
                raise ValueError("global_batch_size is required when dp_size > 1")
            global_batch_size = alive.sum()
        loss = VF.masked_sum(seq, alive) / global_batch_size * dp_size
        if loss_agg_mode == "seq-mean-token-sum-norm":
            loss = loss / (loss_scale_factor if loss_scale_factor is not None else loss_mask.shape[-1])
        return loss
    if loss_agg_mode == "seq-mean-token-mean":
        ntok = torch.sum(loss_mask, dim=-1)
        seq = torch.sum(loss_mat * loss_mask, dim=-1) / (ntok + 1e-8)
        alive = (ntok > 0).float()
        if global_batch_size is None:
            if dp_size > 1:
                raise ValueError("global_batch_size is required when dp_size > 1")
            global_batch_size = alive.sum()
        return VF.masked_sum(seq, alive) / global_batch_size * dp_size
    raise ValueError(f"Invalid loss_agg_mode: {loss_agg_mode}")


def _cfg_get(config, key, default=None):
    if config is None:
        return default
    if hasattr(config, "get"):
        v = config.get(key, default)
    else:
        v = getattr(config, key, default)
    return default if v is None else v


def _global_info(config) -> dict:
    info = _cfg_get(config, "global_batch_info", None)
    return dict(info) if info else {}


def _clip_ranges(config):
    clip = _cfg_get(config, "clip_ratio", 0.2)
    return clip, _cfg_get(config, "clip_ratio_low", clip), _cfg_get(config, "clip_ratio_high", clip)


# ------------------------------------------------------------------------------------------------ policy losses
def compute_policy_loss(old_log_prob, log_prob, advantages, response_mask, cliprange=None, cliprange_low=None,
                        cliprange_high=None, clip_ratio_c=3.0, loss_agg_mode: str = "token-mean"):
    """Functional dual-clip PPO loss (legacy signature). Returns (loss, clipfrac, ppo_kl, clipfrac_lower)."""
    cfg = {"clip_ratio": cliprange, "clip_ratio_low": cliprange_low, "clip_ratio_high": cliprange_high, "clip_ratio_c": clip_ratio_c}
    loss, m = compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, cfg)
    return loss, m["actor/pg_clipfrac"], m["actor/ppo_kl"], m["actor/pg_clipfrac_lower"]


@register_policy_loss("vanilla")
def compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                                config=None, rollout_is_weights=None):
    """PPO clipped surrogate with the dual-clip lower bound for negative advantages."""
    clip, lo, hi = _clip_ranges(config)
    c = _cfg_get(config, "clip_ratio_c", 3.0)
    assert c > 1.0, f"clip_ratio_c must exceed 1.0, got {c}"
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    ppo_kl = VF.masked_mean(-nkl, response_mask)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    lc = torch.maximum(l1, l2)
    clipfrac = VF.masked_mean(torch.gt(l2, l1).float(), response_mask)
    l3 = -advantages * c
    lc2 = torch.min(l3, lc)
    clipfrac_lower = VF.masked_mean(torch.gt(lc, l3) * (advantages < 0).float(), response_mask)
    losses = torch.where(advantages < 0, lc2, lc)
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    return loss, {"actor/pg_clipfrac": clipfrac.detach().item(), "actor/ppo_kl": ppo_kl.detach().item(),
                  "actor/pg_clipfrac_lower": clipfrac_lower.detach().item()}


def _dppo_common(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, config, rollout_is_weights, valid_fn):
    _, lo, hi = _clip_ranges(config)
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    ppo_kl = VF.masked_mean(-nkl, response_mask)
    c = _cfg_get(config, "clip_ratio_c", 20.0)
    trunc = torch.clamp(ratio, max=c).detach()
    prob, old_prob = torch.exp(log_prob), torch.exp(old_log_prob)
    pos_ok, neg_ok = valid_fn(prob, old_prob, log_prob, old_log_prob, lo, hi)
    valid = torch.where(advantages > 0, pos_ok, neg_ok).detach().float()
    losses = -advantages * trunc * log_prob * valid
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    return loss, {"actor/pg_clipfrac": VF.masked_mean(1.0 - valid, response_mask).detach().item(),
                  "actor/ppo_kl": ppo_kl.detach().item(),
                  "actor/pg_clipfrac_lower": VF.masked_mean((ratio > c).float() * valid, response_mask).detach().item()}


@register_policy_loss("dppo_tv")
def compute_policy_loss_dppo_tv(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean", config=None,
                                rollout_is_weights=None):
    """Divergence-PPO, total-variation trust region on the sampled token's probability."""
    def valid(prob, old_prob, lp, olp, lo, hi):
        return (prob - old_prob) <= hi, (prob - old_prob) >= -lo

    return _dppo_common(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, config, rollout_is_weights, valid)


@register_policy_loss("dppo_kl")
def compute_policy_loss_dppo_kl(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean", config=None,
                                rollout_is_weights=None):
    """Divergence-PPO with a binary-KL trust region."""
    def valid(prob, old_prob, lp, olp, lo, hi):
        bkl = old_prob * (olp - lp) + (1 - old_prob) * torch.log((1.0 - old_prob + 1e-8) / (1.0 - prob + 1e-8))
        return (bkl <= hi) | (prob <= old_prob), (bkl <= lo) | (prob >= old_prob)

    return _dppo_common(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, config, rollout_is_weights, valid)


@register_policy_loss("gspo")
def compute_policy_loss_gspo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="seq-mean-token-mean",
                             config=None, rollout_is_weights=None):
    """Sequence-level importance ratio (length-normalised), token-level gradient through the stop-grad trick."""
    _, lo, hi = _clip_ranges(config)
    nkl = log_prob - old_log_prob
    seq_len = torch.sum(response_mask, dim=-1).clamp(min=1)
    nkl_seq = torch.sum(nkl * response_mask, dim=-1) / seq_len
    log_s = torch.clamp(log_prob - log_prob.detach() + nkl_seq.detach().unsqueeze(-1), max=10.0)
    s = torch.exp(log_s)
    l1 = -advantages * s
    l2 = -advantages * torch.clamp(s, 1 - lo, 1 + hi)
    losses = torch.maximum(l1, l2)
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    return loss, {"actor/pg_clipfrac": VF.masked_mean(torch.gt(l2, l1).float(), response_mask).detach().item(),
                  "actor/ppo_kl": VF.masked_mean(-nkl, response_mask).detach().item(), "actor/pg_clipfrac_lower": 0.0}


@register_policy_loss("sapo")
def compute_policy_loss_sapo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="seq-mean-token-mean",
                             config=None, rollout_is_weights=None):
    """Soft adaptive policy optimisation: sigmoid gate σ(τ(r−1))·4/τ with separate τ for ± advantages."""
    tau_pos = torch.as_tensor(_cfg_get(config, "tau_pos", 1.0), dtype=advantages.dtype, device=advantages.device)
    tau_neg = torch.as_tensor(_cfg_get(config, "tau_neg", 1.05), dtype=advantages.dtype, device=advantages.device)
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    taus = torch.where(advantages > 0, tau_pos, tau_neg)
    gates = torch.sigmoid(taus * (ratio - 1.0)) * (4.0 / taus)
    losses = -gates * advantages
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, "seq-mean-token-mean", **_global_info(config))
    return loss, {"actor/pg_clipfrac": 0.0, "actor/ppo_kl": VF.masked_mean(-nkl, response_mask).detach().item(),
                  "actor/pg_clipfrac_lower": 0.0}


@register_policy_loss("gpg")
def compute_policy_loss_gpg(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean", config=None,
                            rollout_is_weights=None):
    losses = -log_prob * advantages
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    return agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config)), {}


@register_policy_loss("clip_cov")
def compute_policy_loss_clip_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                 config=None, rollout_is_weights=None):
    """Clip-Cov: detach a small random subset of tokens whose advantage/log-prob covariance lies in (lb, ub)."""
    pl = _cfg_get(config, "policy_loss", None)
    ratio_cov = _cfg_get(pl, "clip_cov_ratio", 0.0002)
    ub = _cfg_get(pl, "clip_cov_ub", 5.0)
    lb = _cfg_get(pl, "clip_cov_lb", 1.0)
    assert ratio_cov > 0
    _, lo, hi = _clip_ranges(config)
    nkl = log_prob - old_log_prob
    ratio = torch.exp(nkl)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    clipped = (l2 > l1) & (response_mask > 0)
    cov = (advantages - VF.masked_mean(advantages, response_mask)) * (log_prob - VF.masked_mean(log_prob.detach(), response_mask))
    cov = cov.detach().clone()
    cov[response_mask == 0] = -torch.inf
    cov[clipped] = -torch.inf
    n_clip = max(int(ratio_cov * response_mask.sum().item()), 1)
    cand = torch.nonzero((cov < ub) & (cov > lb) & (response_mask > 0))
    corr = torch.ones_like(advantages)
    if len(cand) > 0:
        pick = cand[torch.randperm(len(cand), device=cand.device)[: min(n_clip, len(cand))]]
        corr[pick[:, 0], pick[:, 1]] = 0
    losses = torch.maximum(l1, l2) * corr
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    return loss, {"actor/pg_clipfrac": VF.masked_mean((corr == 0).float(), response_mask).detach().item(),
                  "actor/ppo_kl": VF.masked_mean(-nkl, response_mask).detach().item()}


@register_policy_loss("kl_cov")
def compute_policy_loss_kl_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean", config=None,
                               rollout_is_weights=None):
    """KL-Cov: add |log-ratio| penalty on the top-k% highest-covariance tokens."""
    pl = _cfg_get(config, "policy_loss", None)
    k_ratio = _cfg_get(pl, "kl_cov_ratio", 0.0002)
    coef = _cfg_get(pl, "ppo_kl_coef", 1.0)
    assert k_ratio > 0
    nkl = log_prob - old_log_prob
    ratio = torch.exp(nkl)
    l1 = -advantages * ratio
    lkl = l1 + coef * nkl.abs()
    valid = response_mask > 0
    adv_v, lp_v = advantages[valid].detach(), log_prob[valid].detach()
    sel = torch.zeros_like(valid)
    if adv_v.numel() > 0:
        cov = (adv_v - adv_v.mean()) * (lp_v - lp_v.mean())
        k = max(1, int(cov.numel() * k_ratio))
        top = torch.topk(cov, k, largest=True).indices
        flat_idx = torch.nonzero(valid.reshape(-1)).flatten()[top]
        sel.view(-1)[flat_idx] = True
    losses = torch.where(sel, lkl, l1)
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    return loss, {"actor/ppo_kl": VF.masked_mean(nkl.abs(), response_mask).detach().item()}


@register_policy_loss("geo_mean")
def compute_policy_loss_geo_mean(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                 config=None, rollout_is_weights=None):
    """GMPO: clip token log-ratios, then use the geometric-mean ratio per sequence."""
    _, lo, hi = _clip_ranges(config)
    nkl = log_prob - old_log_prob
    sgn = torch.sign(advantages)
    clamped = torch.clamp(nkl, -lo, hi)
    nkl_min = sgn * torch.min(sgn * nkl, sgn * clamped)
    n = response_mask.sum(dim=-1)
    ratio = torch.exp((nkl_min * response_mask).sum(dim=-1) / (n + 1e-8))
    adv = (advantages * response_mask).sum(dim=-1) / (n + 1e-8)
    losses = -adv * ratio
    if rollout_is_weights is not None:
        losses = losses * torch.exp((torch.log(rollout_is_weights + 1e-10) * response_mask).sum(dim=-1) / (n + 1e-8))
    loss = torch.mean(losses)
    clipped = torch.ne(nkl, clamped)
    return loss, {"actor/pg_clipfrac": VF.masked_mean((clipped * (advantages > 0)).float(), response_mask).detach().item(),
                  "actor/ppo_kl": VF.masked_mean(-nkl, response_mask).detach().item(),
                  "actor/pg_clipfrac_lower": VF.masked_mean((clipped * (advantages < 0)).float(), response_mask).detach().item()}


@register_policy_loss("dro")
def compute_policy_loss_dro(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean", config=None,
                            rollout_is_weights=None):
    """Direct reward optimisation: −(logp·A − β/2·(logp − old)²)."""
    beta = _cfg_get(_cfg_get(config, "policy_loss", None), "dro_beta", None)
    if beta is None or beta <= 0:
        raise ValueError("policy_loss.dro_beta must be a positive value when using DRO")
    lr = log_prob - old_log_prob
    losses = -(log_prob * advantages - 0.5 * beta * lr.square())
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    return loss, {"actor/ppo_kl": VF.masked_mean(-lr, response_mask).detach().item()}


@register_policy_loss("cispo")
def compute_policy_loss_cispo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean", config=None,
                              rollout_is_weights=None):
    """CISPO: clipped, stop-gradient importance weight times the REINFORCE term."""
    _, lo, hi = _clip_ranges(config)
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    clipped = torch.clamp(ratio, 1 - lo, 1 + hi)
    losses = -clipped.detach() * advantages * log_prob
    if rollout_is_weights is not None:
        losses = losses * rollout_is_weights
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    return loss, {"actor/pg_clipfrac": VF.masked_mean((ratio != clipped).float(), response_mask).detach().item(),
                  "actor/ppo_kl": VF.masked_mean(-nkl, response_mask).detach().item(), "actor/pg_clipfrac_lower": 0.0}


def compute_policy_loss_reinforce(rollout_log_prob, log_prob, advantages, response_mask, loss_agg_mode="seq-mean-token-sum",
                                  config=None, rollout_is_weights=None, sc_correction=None):
    """REINFORCE with optional (detached) importance weights: L = −w·logπ·A. ``sc_correction`` is the per-token
    score-centering term (``verl_b200.trainer.ppo.score_centering``), added as ``A · sc_correction`` after the weighting
    (reference: verl/trainer/ppo/core_algos.py:2396-2397)."""
    w = rollout_is_weights if rollout_is_weights is not None else torch.ones_like(advantages)
    losses = -w * log_prob * advantages
    if sc_correction is not None:
        losses = losses + advantages * sc_correction
    loss = agg_loss(losses, response_mask, loss_agg_mode, **_global_info(config))
    nkl = log_prob - rollout_log_prob
    m = {"actor/ppo_kl": VF.masked_mean(-nkl, response_mask).detach().item()}
    if sc_correction is not None:
        m["actor/sc_correction"] = VF.masked_mean(sc_correction.detach(), response_mask).item()
    return loss, m


@register_policy_loss("bypass_mode")
def compute_policy_loss_bypass_mode(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                    config=None, rollout_is_weights=None, sc_correction=None):
    """Bypass mode: ``old_log_prob`` *is* the rollout log-prob (no recompute pass). Importance weights and rejection
    masks between the current policy and the rollout policy are computed on the fly, then either a REINFORCE or a
    PPO-clip objective (``policy_loss.rollout_correction.loss_type``) is applied."""
    from verl_b200.trainer.ppo.rollout_corr_helper import compute_rollout_correction_and_rejection_mask

    pl = _cfg_get(config, "policy_loss", None)
    rc = _cfg_get(pl, "rollout_correction", None) or {}
    loss_type = _cfg_get(rc, "loss_type", "ppo_clip")
    weights, mask, metrics = compute_rollout_correction_and_rejection_mask(
        old_log_prob=log_prob.detach(), rollout_log_prob=old_log_prob, response_mask=response_mask,
        rollout_is=_cfg_get(rc, "rollout_is", None), rollout_is_threshold=_cfg_get(rc, "rollout_is_threshold", 2.0),
        rollout_rs=_cfg_get(rc, "rollout_rs", None), rollout_rs_threshold=_cfg_get(rc, "rollout_rs_threshold", None),
        rollout_is_batch_normalize=_cfg_get(rc, "rollout_is_batch_normalize", False),
    )
    if sc_correction is not None and loss_type != "reinforce":
        raise ValueError("score centering needs policy_loss.rollout_correction.loss_type=reinforce")
    if loss_type == "reinforce":
        loss, m = compute_policy_loss_reinforce(old_log_prob, log_prob, advantages, mask, loss_agg_mode, config, weights, sc_correction)
    else:
        loss, m = compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, mask, loss_agg_mode, config, None)
    m.update(metrics)
    return loss, m


# ------------------------------------------------------------------------------------------------ entropy / value / KL
def compute_entropy_loss(logits, response_mask, loss_agg_mode: str = "token-mean"):
    return agg_loss(VF.entropy_from_logits(logits), response_mask, loss_agg_mode)


def compute_value_loss(vpreds, returns, values, response_mask, cliprange_value: float, loss_agg_mode: str = "token-mean",
                       **global_info):
    """0.5·agg(max((v−R)², (clip(v, v_old ± ε) − R)²)); also returns the clipped fraction."""
    clipped = VF.clip_by_value(vpreds, values - cliprange_value, values + cliprange_value)
    l1 = (vpreds - returns) ** 2
    l2 = (clipped - returns) ** 2
    loss = 0.5 * agg_loss(torch.max(l1, l2), response_mask, loss_agg_mode, **global_info)
    return loss, VF.masked_mean(torch.gt(l2, l1).float(), response_mask)


def kl_penalty_forward(logprob: torch.Tensor, ref_logprob: torch.Tensor, kl_penalty: str) -> torch.Tensor:
    if kl_penalty in ("kl", "k1"):
        return logprob - ref_logprob
    if kl_penalty == "abs":
        return (logprob - ref_logprob).abs()
    if kl_penalty in ("mse", "k2"):
        return 0.5 * (logprob - ref_logprob).square()
    if kl_penalty in ("low_var_kl", "k3"):
        kl = torch.clamp(ref_logprob - logprob, min=-20, max=20)
        return torch.clamp(torch.exp(kl) - kl - 1, min=-10, max=10)
    if kl_penalty == "full":
        raise NotImplementedError("full-distribution KL needs the logits of both policies")
    raise NotImplementedError(f"unknown kl penalty {kl_penalty}")


def kl_penalty(logprob: torch.Tensor, ref_logprob: torch.Tensor, kl_penalty: str) -> torch.Tensor:
    """Per-token KL estimate. A trailing ``+`` (e.g. ``k3+``) keeps the value of that estimator but routes the
    gradient through the k2 estimator (unbiased gradient, straight-through)."""
    fwd = kl_penalty_forward(logprob, ref_logprob, kl_penalty.rstrip("+"))
    if not kl_penalty.endswith("+") or kl_penalty in ("mse+", "k2+"):
        return fwd
    bwd = kl_penalty_forward(logprob, ref_logprob, "k2")
    return bwd - bwd.detach() + fwd.detach()


def compute_pf_ppo_reweight_data(data, reweight_method: str = "pow", weight_pow: float = 2.0):
    """PF-PPO: resample the batch with replacement, weights derived from sequence scores."""
    from copy import deepcopy

    from verl_b200.protocol import TensorBatch

    scores = data.batch["token_level_scores"].sum(dim=-1)
    if reweight_method == "pow":
        w = torch.pow(torch.abs(scores), weight_pow)
    elif reweight_method == "max_min":
        w = torch.where((scores == scores.max()) | (scores == scores.min()), 1.0, 0.0)
    elif reweight_method == "max_random":
        w = torch.where(scores == scores.max(), 0.4, 0.1)
    else:
        raise ValueError(f"Unsupported reweight_method: {reweight_method}")
    w = torch.clamp(w + 1e-8, min=1e-8)
    n = scores.shape[0]
    idx = torch.multinomial(w, n, replacement=True)
    out = deepcopy(data)
    out.batch = TensorBatch({k: v[idx] for k, v in data.batch.items()}, batch_size=data.batch.batch_size)
    idx_np = idx.cpu().numpy()
    out.non_tensor_batch = {k: v[idx_np] for k, v in data.non_tensor_batch.items()}
    out.meta_info = {k: ([v[i] for i in idx_np] if isinstance(v, list) and len(v) == n else v) for k, v in data.meta_info.items()}
    return out
