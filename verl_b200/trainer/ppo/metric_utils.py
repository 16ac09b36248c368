"""Training metrics: data statistics, timing, throughput, validation aggregation.

Parity target: ``verl/trainer/ppo/metric_utils.py`` (compute_data_metrics :429, compute_timing_metrics :611,
compute_throughout_metrics :655, compute_variance_proxy_metrics :691, process_validation_metrics :805, bootstrap_metric,
calc_maj_val) and ``reduce_metrics`` re-export.
"""

from __future__ import annotations

from collections import defaultdict
from functools import partial
from typing import Any, Callable, Optional

import numpy as np
import torch

from verl_b200.protocol import DataProto
from verl_b200.utils import torch_functional as VF
from verl_b200.utils.metric import reduce_metrics  # noqa: F401

__all__ = ["reduce_metrics", "compute_data_metrics", "compute_timing_metrics", "compute_throughout_metrics",
           "compute_variance_proxy_metrics", "bootstrap_metric", "calc_maj_val", "process_validation_metrics",
           "_compute_response_info"]


def _compute_response_info(batch: DataProto) -> dict[str, Any]:
    R = batch.batch["responses"].shape[-1]
    att = batch.batch["attention_mask"]
    prompt_mask, response_mask = att[:, :-R], att[:, -R:]
    return {"response_mask": response_mask, "prompt_length": prompt_mask.sum(-1).float(), "response_length": response_mask.sum(-1).float()}


def compute_data_metrics(batch: DataProto, use_critic: bool = True) -> dict[str, Any]:
    b = batch.batch
    seq_score = b["token_level_scores"].sum(-1)
    seq_reward = b["token_level_rewards"].sum(-1)
    adv, ret = b["advantages"], b["returns"]
    R = b["responses"].shape[-1]
    max_prompt = b["attention_mask"].shape[-1] - R
    info = _compute_response_info(batch)
    prompt_len, resp_len = info["prompt_length"], info["response_length"]
    rmask = (b["response_mask"] if "response_mask" in b else info["response_mask"]).bool()
    aborted = resp_len == 0
    non_aborted = ~aborted
    valid_adv, valid_ret = torch.masked_select(adv, rmask), torch.masked_select(ret, rmask)
    nz = lambda t, fn: fn(t).detach().item() if t.numel() else 0.0
    m = {
        "critic/score/mean": nz(seq_score[non_aborted], torch.mean), "critic/score/max": nz(seq_score[non_aborted], torch.max),
        "critic/score/min": nz(seq_score[non_aborted], torch.min),
        "critic/rewards/mean": nz(seq_reward[non_aborted], torch.mean), "critic/rewards/max": nz(seq_reward[non_aborted], torch.max),
        "critic/rewards/min": nz(seq_reward[non_aborted], torch.min),
        "critic/advantages/mean": nz(valid_adv, torch.mean), "critic/advantages/max": nz(valid_adv, torch.max),
        "critic/advantages/min": nz(valid_adv, torch.min),
        "critic/returns/mean": nz(valid_ret, torch.mean), "critic/returns/max": nz(valid_ret, torch.max),
        "critic/returns/min": nz(valid_ret, torch.min),
    }
    if use_critic and "values" in b:
        vals = torch.masked_select(b["values"], rmask)
        ret_diff_var = torch.var(valid_ret - vals) if vals.numel() > 1 else torch.tensor(0.0)
        ret_var = torch.var(valid_ret) if valid_ret.numel() > 1 else torch.tensor(1.0)
        m.update({"critic/values/mean": nz(vals, torch.mean), "critic/values/max": nz(vals, torch.max), "critic/values/min": nz(vals, torch.min),
                  "critic/vf_explained_var": (1.0 - ret_diff_var / (ret_var + 1e-5)).detach().item()})
    rl = resp_len[non_aborted]
    m.update({
        "response_length/mean": nz(resp_len, torch.mean), "response_length/max": nz(resp_len, torch.max), "response_length/min": nz(resp_len, torch.min),
        "response_length/clip_ratio": torch.mean(torch.eq(resp_len, R).float()).item(),
        "response_length_non_aborted/mean": nz(rl, torch.mean), "response_length_non_aborted/max": nz(rl, torch.max),
        "response_length_non_aborted/min": nz(rl, torch.min),
        "response_length_non_aborted/clip_ratio": torch.mean(torch.eq(rl, R).float()).item() if rl.numel() else 0.0,
        "response/aborted_ratio": aborted.float().mean().item(),
        "prompt_length/mean": nz(prompt_len, torch.mean), "prompt_length/max": nz(prompt_len, torch.max), "prompt_length/min": nz(prompt_len, torch.min),
        "prompt_length/clip_ratio": torch.mean(torch.eq(prompt_len, max_prompt).float()).item(),
    })
    if "__num_turns__" in batch.non_tensor_batch:
        nt = np.asarray(batch.non_tensor_batch["__num_turns__"], dtype=np.float64)
        m.update({"num_turns/min": nt.min(), "num_turns/max": nt.max(), "num_turns/mean": nt.mean()})
    if "tool_call_counts" in batch.non_tensor_batch:
        tc = np.asarray(batch.non_tensor_batch["tool_call_counts"], dtype=np.float64)
        m.update({"tool_call_counts/min": tc.min(), "tool_call_counts/max": tc.max(), "tool_call_counts/mean": tc.mean()})
    return m


def compute_timing_metrics(batch: DataProto, timing_raw: dict[str, float]) -> dict[str, Any]:
    info = _compute_response_info(batch)
    n_prompt = torch.sum(info["prompt_length"]).item()
    n_resp = torch.sum(info["response_length"]).item()
    n_all = n_prompt + n_resp
    per_section = {"gen": n_resp, **{k: n_all for k in ("ref", "values", "adv", "update_critic", "update_actor", "old_log_prob")}}
    out = {f"timing_s/{k}": v for k, v in timing_raw.items()}
    out.update({f"timing_per_token_ms/{k}": timing_raw[k] * 1000 / max(per_section[k], 1) for k in set(per_section) & set(timing_raw)})
    return out


def compute_throughout_metrics(batch: DataProto, timing_raw: dict[str, float], n_gpus: int) -> dict[str, Any]:
    """``perf/throughput`` = tokens (prompt + response over the global batch) per second per GPU."""
    total = sum(batch.meta_info["global_token_num"])
    t = timing_raw["step"]
    return {"perf/total_num_tokens": total, "perf/time_per_step": t, "perf/throughput": total / (t * n_gpus)}


def compute_variance_proxy_metrics(batch: DataProto, gradient_norm: float | None = None) -> dict[str, float]:
    """Cheap proxies of policy-gradient variance: advantage second moment and, with Σπ², the score-function norm."""
    m = {}
    b = batch.batch
    if "advantages" not in b:
        return m
    mask = b["response_mask"].float()
    adv = b["advantages"]
    m["variance_proxy/adv_sq_mean"] = VF.masked_mean(adv**2, mask).item()
    if "sum_pi_squared" in b and "old_log_probs" in b:
        w = 1 - 2 * torch.exp(b["old_log_probs"]) + b["sum_pi_squared"]
        m["variance_proxy/score_norm_sq_mean"] = VF.masked_mean(w, mask).item()
        m["variance_proxy/proxy1_signal_strength"] = VF.masked_mean(adv**2 * w, mask).item()
    if gradient_norm is not None:
        m["variance_proxy/grad_norm_sq"] = float(gradient_norm) ** 2
    return m


def bootstrap_metric(data: list, subset_size: int, reduce_fns: list[Callable], n_bootstrap: int = 1000, seed: int = 42):
    """[(mean, std)] of each reduce function over ``n_bootstrap`` resamples of ``subset_size`` items."""
    rng = np.random.RandomState(seed)
    res = [[] for _ in reduce_fns]
    for _ in range(n_bootstrap):
        idx = rng.choice(len(data), size=subset_size, replace=True)
        sample = [data[i] for i in idx]
        for i, fn in enumerate(reduce_fns):
            res[i].append(fn(sample))
    return [(float(np.mean(r)), float(np.std(r))) for r in res]


def calc_maj_val(data: list[dict], vote_key: str, val_key: str) -> float:
    """Value of the majority-voted answer."""
    groups = defaultdict(list)
    for d in data:
        groups[d[vote_key]].append(d[val_key])
    winner = max(groups.items(), key=lambda kv: len(kv[1]))[0]
    return groups[winner][0]


def process_validation_metrics(data_sources: list[str], sample_uids: list[str], infos_dict: dict[str, list], seed: int = 42):
    """``{data_source: {var: {"mean@N" | "std@N" | "best@k/mean" | "worst@k/mean" | "maj@k/mean": value}}}``."""
    by_src = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    for i, src in enumerate(data_sources):
        for var, vals in infos_dict.items():
            by_src[src][sample_uids[i]][var].append(vals[i])
    out = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    for src, by_uid in by_src.items():
        for uid, var2vals in by_uid.items():
            for var, vals in var2vals.items():
                if not vals or isinstance(vals[0], str):
                    continue
                n = len(vals)
                metric = {f"mean@{n}": float(np.mean(vals))}
                if n > 1:
                    metric[f"std@{n}"] = float(np.std(vals))
                    ns = []
                    k = 2
                    while k < n:
                        ns.append(k)
                        k *= 2
                    ns.append(n)
                    for k in ns:
                        (bm, bs), (wm, ws) = bootstrap_metric(vals, k, [np.max, np.min], seed=seed)
                        metric[f"best@{k}/mean"], metric[f"best@{k}/std"] = bm, bs
                        metric[f"worst@{k}/mean"], metric[f"worst@{k}/std"] = wm, ws
                        if var2vals.get("pred") is not None:
                            vote = [{"val": v, "pred": p} for v, p in zip(vals, var2vals["pred"])]
                            [(mm, ms)] = bootstrap_metric(vote, k, [partial(calc_maj_val, vote_key="pred", val_key="val")], seed=seed)
                            metric[f"maj@{k}/mean"], metric[f"maj@{k}/std"] = mm, ms
                for name, v in metric.items():
                    out[src][var][name].append(v)
    return {src: {var: {name: float(np.mean(v)) for name, v in d.items()} for var, d in vd.items()} for src, vd in out.items()}


# ------------------------------------------------------------------------------------------------ rollout MoE load balance
def rollout_moe_load_counts(routed_experts, response_mask, num_experts: Optional[int]):
    """``[layers, experts]`` counts of the experts chosen for the RESPONSE tokens of a batch.

    ``routed_experts`` is ``[bs, seq, layers, topk]`` (what router replay R3 carries), ``response_mask`` ``[bs, R]``. Each
    sequence's last response token is left out: it was sampled but never fed to the model, its row is a filler. Returns
    ``None`` when nothing can be counted (missing inputs, ids outside ``[0, num_experts)``).
    Reference: ``verl/trainer/ppo/metric_utils.py:205-272``."""
    if routed_experts is None or response_mask is None or not num_experts or num_experts <= 0:
        return None
    if routed_experts.dim() != 4 or response_mask.dim() != 2 or response_mask.shape[0] != routed_experts.shape[0]:
        return None
    R = response_mask.shape[1]
    if R == 0 or routed_experts.shape[1] < R:
        return None
    mask = response_mask.bool().clone()
    n_valid = mask.sum(-1)
    rows = torch.nonzero(n_valid > 0, as_tuple=True)[0]
    if rows.numel():
        pos = torch.arange(R, device=mask.device).expand_as(mask)
        last = torch.where(mask, pos, torch.full_like(pos, -1)).amax(-1)
        mask[rows, last[rows]] = False
    picked = routed_experts[:, -R:][mask.to(routed_experts.device)].long().cpu()          # [tokens, layers, topk]
    if picked.numel() == 0 or int(picked.min()) < 0 or int(picked.max()) >= num_experts:
        return None
    L = picked.shape[1]
    flat = picked + torch.arange(L).view(1, L, 1) * num_experts                            # one bincount over (layer, expert)
    return torch.bincount(flat.reshape(-1), minlength=L * num_experts).view(L, num_experts)


def moe_load_balance_metrics(load_counts, prefix: str = "rollout/moe") -> dict:
    """Violation of a uniform load per layer: with ``f_e`` the fraction of assignments that went to expert ``e`` and ``E``
    experts, ``dev_e = f_e·E − 1``; ``max_vio`` / ``min_vio`` are the extremes, ``avg_vio`` the mean absolute deviation.
    Per-layer values plus max / avg over layers (reference ``metric_utils.py:176-202``)."""
    if load_counts is None or load_counts.numel() == 0:
        return {}
    frac = load_counts.float()
    frac = frac / frac.sum(1, keepdim=True).clamp_min(1.0)
    dev = frac * frac.shape[1] - 1.0
    stats = {"max_vio": dev.max(1).values, "min_vio": dev.min(1).values, "avg_vio": dev.abs().mean(1)}
    out = {}
    for name, v in stats.items():
        for i, x in enumerate(v.tolist()):
            out[f"{prefix}/{name}/layer_{i}"] = x
        out[f"{prefix}/{name}/max"] = float(v.max())
        out[f"{prefix}/{name}/avg"] = float(v.mean())
    return out


def compute_rollout_moe_load_balance_metrics(routed_experts, response_mask, num_experts, prefix: str = "rollout/moe") -> dict:
    return moe_load_balance_metrics(rollout_moe_load_counts(routed_experts, response_mask, num_experts), prefix)


class RolloutMoELoadBalanceMetricsAccumulator:
    """Sums the routed-expert counts of several steps and reports them every ``interval`` steps
    (``trainer.moe_lb_metrics_interval``; reference ``metric_utils.py:312-427``)."""

    def __init__(self, num_experts: Optional[int] = None):
        self.num_experts = num_experts
        self.load_counts = None

    def update(self, routed_experts, response_mask, num_experts: Optional[int] = None) -> bool:
        c = rollout_moe_load_counts(routed_experts, response_mask, num_experts or self.num_experts)
        if c is None:
            return False
        self.load_counts = c if self.load_counts is None or self.load_counts.shape != c.shape else self.load_counts + c
        return True

    def total_assignments(self) -> int:
        return 0 if self.load_counts is None else int(self.load_counts.sum())

    def pop_metrics(self, prefix: str = "rollout/moe") -> dict:
        m = moe_load_balance_metrics(self.load_counts, prefix)
        self.load_counts = None
        return m


def compute_moe_lb_metrics(batch: DataProto, interval: int, global_steps: int, accumulator: RolloutMoELoadBalanceMetricsAccumulator) -> dict:
    """Feed one step's batch to the accumulator; on every ``interval``-th step return (and reset) the accumulated metrics."""
    if interval <= 0:
        return {}
    accumulator.update(batch.batch.get("routed_experts", None), batch.batch.get("response_mask", None))
    if global_steps % interval != 0:
        return {}
    n = accumulator.total_assignments()
    m = accumulator.pop_metrics()
    m["rollout/moe/routed_experts_found"] = float(n > 0)
    m["rollout/moe/routed_expert_assignments"] = n
    return m


# ------------------------------------------------------------------------------------------------ speculative decoding
def compute_spec_decode_metrics(spec_drafts, spec_accepts, spec_verifies, non_padding_mask=None) -> dict:
    """Per-request acceptance statistics of speculative decoding, averaged with equal weight per request:
    ``accept_rate = accepted / drafted`` and ``accept_length = 1 + accepted / verify_steps`` (0 where the denominator is 0).
    The three inputs are per-request counters reported by the rollout engine (all ``None`` = feature off → ``{}``).
    Reference: ``verl/trainer/ppo/ray_trainer.py:138-184``."""
    given = [x is not None for x in (spec_drafts, spec_accepts, spec_verifies)]
    if not any(given):
        return {}
    assert all(given), "spec-decode metrics need drafted, accepted and verify-step counters together"
    cols = [list(x.tolist() if hasattr(x, "tolist") else x) for x in (spec_drafts, spec_accepts, spec_verifies)]
    if non_padding_mask is not None:
        keep = [bool(k) for k in non_padding_mask]
        assert len(keep) == len(cols[0])
        cols = [[v for v, k in zip(c, keep) if k] for c in cols]
    d, a, v = cols
    if not d:
        return {}
    rate = [ai / di if di > 0 else 0.0 for ai, di in zip(a, d)]
    length = [1.0 + ai / vi if vi > 0 else 0.0 for ai, vi in zip(a, v)]
    return {"rollout/spec_accept_rate": float(sum(rate) / len(rate)), "rollout/spec_accept_length": float(sum(length) / len(length))}
