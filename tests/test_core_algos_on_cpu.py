import math

import numpy as np
import pytest
import torch

from verl_b200.trainer.ppo import core_algos as ca
from verl_b200.utils import torch_functional as VF


def test_registries():
    for n in ["gae", "grpo", "rloo", "reinforce_plus_plus", "remax", "opo", "gpg", "gdpo", "grpo_passk", "rloo_vectorized",
              "grpo_vectorized", "reinforce_plus_plus_baseline", "optimal_token_baseline", "tir_optimal_token_baseline"]:
        assert callable(ca.get_adv_estimator_fn(n))
    for n in ["vanilla", "dppo_tv", "dppo_kl", "gspo", "sapo", "gpg", "clip_cov", "kl_cov", "geo_mean", "dro", "cispo", "bypass_mode"]:
        assert callable(ca.get_policy_loss_fn(n))
    with pytest.raises(ValueError):
        ca.get_adv_estimator_fn("nope")


def _grpo_loop(scores, index, eps=1e-6):
    out = torch.zeros_like(scores)
    groups = {}
    for i, g in enumerate(index):
        groups.setdefault(g, []).append(i)
    for g, idx in groups.items():
        s = scores[idx]
        mean, std = (torch.tensor(0.0), torch.tensor(1.0)) if len(idx) == 1 else (s.mean(), s.std())
        out[idx] = (s - mean) / (std + eps)
    return out


def test_grpo_matches_per_group_loop():
    torch.manual_seed(0)
    bs, L = 12, 7
    mask = (torch.rand(bs, L) > 0.3).float()
    mask[:, 0] = 1
    rew = torch.zeros(bs, L)
    rew[torch.arange(bs), (mask.sum(-1) - 1).long()] = torch.randn(bs)
    index = np.array(["a", "a", "a", "b", "b", "c", "d", "d", "d", "d", "e", "e"], dtype=object)
    adv, ret = ca.compute_grpo_outcome_advantage(rew, mask, index)
    ref = _grpo_loop(rew.sum(-1), index).unsqueeze(-1) * mask
    assert torch.allclose(adv, ref, atol=1e-6) and torch.equal(adv, ret)
    adv2, _ = ca.compute_grpo_outcome_advantage(rew, mask, index, norm_adv_by_std_in_grpo=False)
    s = rew.sum(-1)
    assert math.isclose(adv2[0, 0].item(), (s[0] - s[:3].mean()).item(), rel_tol=1e-5)


def test_rloo_and_opo_and_gpg():
    rew = torch.zeros(4, 3)
    rew[:, 2] = torch.tensor([1.0, 0.0, 2.0, 5.0])
    mask = torch.ones(4, 3)
    idx = np.array([0, 0, 0, 1])
    adv, _ = ca.compute_rloo_outcome_advantage(rew, mask, idx)
    assert torch.allclose(adv[:, 0], torch.tensor([1 - 1.0, 0 - 1.5, 2 - 0.5, 5.0]))
    adv_o, _ = ca.compute_opo_outcome_advantage(rew, mask, idx)
    assert torch.allclose(adv_o[:3, 0], torch.tensor([0.0, -1.0, 1.0])) and adv_o[3, 0] == 5.0
    adv_g, _ = ca.compute_gpg_outcome_advantage(rew, mask, idx)
    alpha = 4 / 3
    assert torch.allclose(adv_g[:3, 0], alpha * torch.tensor([0.0, -1.0, 1.0]))


def test_gae_simple():
    rew = torch.tensor([[0.0, 0.0, 1.0]])
    val = torch.tensor([[0.5, 0.5, 0.5]])
    mask = torch.ones(1, 3)
    with torch.no_grad():
        adv, ret = ca.compute_gae_advantage_return(rew, val, mask, gamma=1.0, lam=1.0)
    assert torch.allclose(ret, torch.tensor([[1.0, 1.0, 1.0]]))
    # masked position in the middle is skipped: its return still follows the carried state
    mask2 = torch.tensor([[1.0, 0.0, 1.0]])
    adv2, ret2 = ca.compute_gae_advantage_return(rew, val, mask2, 1.0, 1.0)
    assert math.isclose(ret2[0, 0].item(), 1.0, rel_tol=1e-5)


def test_remax_and_reinforce_pp():
    rew = torch.tensor([[0.0, 1.0, 0.0], [1.0, 0.0, 0.0]])
    mask = torch.tensor([[1.0, 1.0, 0.0], [1.0, 1.0, 1.0]])
    adv, ret = ca.compute_remax_outcome_advantage(rew, torch.tensor([0.5, 0.25]), mask)
    assert torch.allclose(ret, torch.tensor([[1.0, 1.0, 0.0], [1.0, 0.0, 0.0]]))
    assert torch.allclose(adv[0], torch.tensor([0.5, 0.5, 0.0]))
    adv2, ret2 = ca.compute_reinforce_plus_plus_outcome_advantage(rew, mask, gamma=0.5)
    assert math.isclose(ret2[0, 0].item(), 0.5, rel_tol=1e-6)


def test_passk():
    rew = torch.zeros(4, 2)
    rew[:, 1] = torch.tensor([1.0, 3.0, 2.0, 0.0])
    mask = torch.ones(4, 2)
    adv, _ = ca.compute_grpo_passk_outcome_advantage(rew, mask, np.array([0, 0, 0, 0]), norm_adv_by_std_in_grpo=False)
    assert adv[:, 0].tolist() == [0.0, 1.0, 0.0, 0.0]


@pytest.mark.parametrize("mode", ["token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm", "token-sum"])
def test_agg_loss_invariant_to_dp_and_micro_split(mode):
    """Sum of micro-batch losses, averaged over DP ranks, equals the loss of the whole batch."""
    torch.manual_seed(1)
    bs, L = 8, 6
    mat = torch.randn(bs, L)
    mask = (torch.rand(bs, L) > 0.4).float()
    mask[:, 0] = 1
    whole = ca.agg_loss(mat, mask, mode)
    dp = 2
    info = dict(dp_size=dp, batch_num_tokens=mask.sum(), global_batch_size=float(bs))
    per_rank = []
    for r in range(dp):
        rm, rk = mat[r * 4:(r + 1) * 4], mask[r * 4:(r + 1) * 4]
        per_rank.append(sum(ca.agg_loss(rm[i:i + 2], rk[i:i + 2], mode, **info) for i in (0, 2)))
    assert torch.allclose(torch.stack(per_rank).mean(), whole, atol=1e-5)


def test_vanilla_ppo_clip_and_dual_clip():
    old = torch.zeros(1, 4)
    new = torch.log(torch.tensor([[1.5, 0.5, 5.0, 1.0]]))
    adv = torch.tensor([[1.0, 1.0, -1.0, -1.0]])
    mask = torch.ones(1, 4)
    loss, m = ca.compute_policy_loss_vanilla(old, new, adv, mask, "token-mean", {"clip_ratio": 0.2, "clip_ratio_c": 3.0})
    # per token: -min(1.5,1.2)= -1.2 ; -0.5 ; dual clip min(3, 5)=3 ; 1.0
    assert math.isclose(loss.item(), (-1.2 - 0.5 + 3.0 + 1.0) / 4, rel_tol=1e-5)
    assert math.isclose(m["actor/pg_clipfrac"], 0.25, rel_tol=1e-6) and math.isclose(m["actor/pg_clipfrac_lower"], 0.25, rel_tol=1e-6)


@pytest.mark.parametrize("name", ["vanilla", "dppo_tv", "dppo_kl", "gspo", "sapo", "gpg", "clip_cov", "kl_cov", "geo_mean", "cispo"])
def test_policy_losses_run_and_backprop(name):
    torch.manual_seed(0)
    old = -torch.rand(4, 5) - 0.1
    new = (old + 0.05 * torch.randn(4, 5)).requires_grad_(True)
    adv = torch.randn(4, 5)
    mask = torch.ones(4, 5)
    cfg = {"clip_ratio": 0.2, "clip_ratio_low": 0.2, "clip_ratio_high": 0.28, "clip_ratio_c": 3.0, "tau_pos": 1.0, "tau_neg": 1.05,
           "policy_loss": {"clip_cov_ratio": 0.1, "clip_cov_lb": -10.0, "clip_cov_ub": 10.0, "kl_cov_ratio": 0.2, "ppo_kl_coef": 1.0}}
    loss, metrics = ca.get_policy_loss_fn(name)(old, new, adv, mask, "token-mean", cfg)
    loss.backward()
    assert torch.isfinite(loss) and new.grad is not None and torch.isfinite(new.grad).all()


def test_dro_requires_beta():
    with pytest.raises(ValueError):
        ca.compute_policy_loss_dro(torch.zeros(1, 2), torch.zeros(1, 2), torch.ones(1, 2), torch.ones(1, 2), config={"policy_loss": {}})
    l, _ = ca.compute_policy_loss_dro(torch.zeros(1, 2), torch.full((1, 2), 0.1), torch.ones(1, 2), torch.ones(1, 2), config={"policy_loss": {"dro_beta": 2.0}})
    assert math.isclose(l.item(), -(0.1 - 0.5 * 2.0 * 0.01), rel_tol=1e-5)


def test_kl_penalties():
    lp, ref = torch.tensor([[-1.0, -2.0]]), torch.tensor([[-1.5, -1.0]])
    assert torch.allclose(ca.kl_penalty(lp, ref, "kl"), lp - ref)
    assert torch.allclose(ca.kl_penalty(lp, ref, "abs"), (lp - ref).abs())
    assert torch.allclose(ca.kl_penalty(lp, ref, "mse"), 0.5 * (lp - ref) ** 2)
    k = ref - lp
    assert torch.allclose(ca.kl_penalty(lp, ref, "low_var_kl"), torch.exp(k) - k - 1)
    lpg = lp.clone().requires_grad_(True)
    v = ca.kl_penalty(lpg, ref, "k3+")
    assert torch.allclose(v, ca.kl_penalty(lp, ref, "k3"))
    v.sum().backward()
    assert torch.allclose(lpg.grad, (lp - ref))   # gradient of the k2 estimator


def test_value_loss_and_kl_controller():
    v, r, old = torch.tensor([[1.0, 3.0]]), torch.tensor([[0.0, 0.0]]), torch.tensor([[0.0, 0.0]])
    loss, frac = ca.compute_value_loss(v, r, old, torch.ones(1, 2), cliprange_value=0.5)
    assert math.isclose(loss.item(), 0.5 * (1.0 + 9.0) / 2, rel_tol=1e-6) and frac.item() == 0.0
    c = ca.AdaptiveKLController(0.1, target_kl=0.1, horizon=100)
    c.update(0.2, 10)
    assert math.isclose(c.value, 0.1 * (1 + 0.2 * 10 / 100))
    f = ca.get_kl_controller({"type": "fixed", "kl_coef": 0.3})
    f.update(1.0, 1)
    assert f.value == 0.3


def test_masked_helpers():
    x = torch.tensor([[1.0, 2.0, 3.0]])
    m = torch.tensor([[1.0, 0.0, 1.0]])
    assert VF.masked_mean(x, m).item() == pytest.approx(2.0)
    w = VF.masked_whiten(torch.tensor([[1.0, 5.0, 3.0, 9.0]]), torch.tensor([[1.0, 1.0, 1.0, 0.0]]))
    assert abs(VF.masked_mean(w, torch.tensor([[1.0, 1.0, 1.0, 0.0]])).item()) < 1e-6
    assert VF.get_response_mask(torch.tensor([[5, 2, 7, 2]]), eos_token=2).tolist() == [[1, 1, 0, 0]]


def test_optimal_token_baseline_shapes():
    torch.manual_seed(0)
    bs, L = 6, 5
    rew = torch.zeros(bs, L)
    rew[:, -1] = torch.randn(bs)
    mask = torch.ones(bs, L)
    idx = np.array([0, 0, 0, 1, 1, 2])
    olp = -torch.rand(bs, L)
    spi = torch.rand(bs, L)
    adv, ret = ca.compute_optimal_token_baseline_advantage(rew, mask, idx, olp, spi)
    assert adv.shape == (bs, L) and torch.allclose(adv[5], ret[5])   # singleton group: no baseline
    adv2, _ = ca.compute_multi_turn_optimal_token_baseline_advantage(rew, mask, idx, olp, spi)
    assert torch.isfinite(adv2).all()


def test_moe_load_balance_and_spec_decode_metrics():
    import torch

    from verl_b200.trainer.ppo.metric_utils import (RolloutMoELoadBalanceMetricsAccumulator, compute_rollout_moe_load_balance_metrics,
                                                    compute_spec_decode_metrics, rollout_moe_load_counts)

    bs, P, R, L, k, E = 2, 3, 4, 2, 2, 4
    routed = torch.zeros(bs, P + R, L, k, dtype=torch.int16)
    routed[:, :, 0] = torch.tensor([0, 1])                  # layer 0: always experts 0 and 1
    routed[:, :, 1, 0] = torch.arange(P + R) % E             # layer 1: slot 0 cycles, slot 1 fixed on expert 3
    routed[:, :, 1, 1] = 3
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 1, 1]])
    counts = rollout_moe_load_counts(routed, mask, E)
    # sequence 0 contributes 2 response tokens (its 3rd = last valid is dropped), sequence 1 contributes 3
    assert counts.shape == (L, E) and counts[0].tolist() == [5, 5, 0, 0] and int(counts.sum()) == 5 * L * k
    m = compute_rollout_moe_load_balance_metrics(routed, mask, E)
    assert m["rollout/moe/max_vio/layer_0"] == pytest.approx(1.0) and m["rollout/moe/min_vio/layer_0"] == pytest.approx(-1.0)
    assert m["rollout/moe/avg_vio/layer_0"] == pytest.approx(1.0) and "rollout/moe/max_vio/avg" in m
    assert rollout_moe_load_counts(routed + 10, mask, E) is None and compute_rollout_moe_load_balance_metrics(None, mask, E) == {}
    acc = RolloutMoELoadBalanceMetricsAccumulator(E)
    assert acc.update(routed, mask) and acc.update(routed, mask) and acc.total_assignments() == 2 * int(counts.sum())
    assert acc.pop_metrics()["rollout/moe/max_vio/layer_0"] == pytest.approx(1.0) and acc.total_assignments() == 0

    assert compute_spec_decode_metrics(None, None, None) == {}
    s = compute_spec_decode_metrics([10, 0, 8], [5, 0, 8], [5, 0, 4], non_padding_mask=[True, True, True])
    assert s["rollout/spec_accept_rate"] == pytest.approx((0.5 + 0 + 1.0) / 3) and s["rollout/spec_accept_length"] == pytest.approx((2 + 0 + 3) / 3)
    with pytest.raises(AssertionError):
        compute_spec_decode_metrics([1], None, None)
