"""Fused PPO loss / GRPO advantage kernels against the PyTorch formulations of the algorithm layer."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("agg", ["token-mean", "seq-mean-token-mean", "seq-mean-token-sum"])
@pytest.mark.parametrize("kl", [None, "low_var_kl", "mse"])
def test_fused_ppo_loss_matches_core_algos(agg, kl):
    from verl_b200.trainer.ppo import core_algos
    from verl_b200.workers.utils.losses import ppo_loss

    torch.manual_seed(0)
    bs, R = 12, 77
    old = -2 + 0.5 * torch.randn(bs, R, device="cuda")
    lp = (old + 0.3 * torch.randn(bs, R, device="cuda")).requires_grad_(True)
    ref = old + 0.2 * torch.randn(bs, R, device="cuda")
    adv = torch.randn(bs, R, device="cuda") * 2
    mask = (torch.rand(bs, R, device="cuda") > 0.2).float()
    mask[3] = 0
    cfg = {"clip_ratio": 0.2, "clip_ratio_low": 0.2, "clip_ratio_high": 0.28, "clip_ratio_c": 3.0, "loss_agg_mode": agg, "use_kl_loss": kl is not None,
           "kl_loss_type": kl or "low_var_kl", "kl_loss_coef": 0.05, "entropy_coeff": 0.0, "policy_loss": {"loss_mode": "vanilla"}}
    data = {"old_log_probs": old, "advantages": adv, "response_mask": mask, "ref_log_prob": ref, "dp_size": 2,
            "batch_num_tokens": mask.sum() * 2, "global_batch_size": torch.tensor(22.0, device="cuda")}
    loss, m = ppo_loss(cfg, {"log_probs": lp}, data)
    (g,) = torch.autograd.grad(loss, lp)
    # reference: the unfused formulation
    lp2 = lp.detach().clone().requires_grad_(True)
    info = {"dp_size": 2, "batch_num_tokens": data["batch_num_tokens"], "global_batch_size": data["global_batch_size"]}
    view = dict(cfg, global_batch_info=info)
    pg, pm = core_algos.compute_policy_loss_vanilla(old, lp2, adv, mask, agg, type("C", (dict,), {"__getattr__": dict.__getitem__})(view))
    ref_loss = pg
    if kl:
        ref_loss = ref_loss + 0.05 * core_algos.agg_loss(core_algos.kl_penalty(lp2, ref, kl), mask, agg, **info)
    (g2,) = torch.autograd.grad(ref_loss, lp2)
    torch.testing.assert_close(loss, ref_loss, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(g, g2, rtol=1e-4, atol=1e-7)
    assert abs(m["actor/pg_clipfrac"].aggregate() - pm["actor/pg_clipfrac"]) < 1e-5
    assert abs(m["actor/ppo_kl"].aggregate() - pm["actor/ppo_kl"]) < 1e-5


def test_grpo_advantage_kernel():
    from verl_b200.ops.rl import grpo_advantage
    from verl_b200.trainer.ppo import core_algos
    import numpy as np

    torch.manual_seed(1)
    B, R, n = 48, 33, 8
    rewards = torch.zeros(B, R)
    mask = (torch.rand(B, R) > 0.3).float()
    mask[:, 0] = 1
    sc = torch.randint(0, 2, (B,)).float()
    for b in range(B):
        last = int(mask[b].nonzero().max())
        rewards[b, last] = sc[b]
    gidx = torch.arange(B) // n
    gidx[-1] = 99                                    # a singleton group
    uid = np.array([str(int(g)) for g in gidx], dtype=object)
    want, _ = core_algos.compute_grpo_outcome_advantage(rewards, mask, uid)
    from verl_b200.utils.groupwise import as_torch_index

    got = grpo_advantage(rewards.sum(-1).cuda(), as_torch_index(uid).cuda(), mask.cuda())
    torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-5)


def test_grouped_gemm_matches_per_expert_loop():
    from verl_b200.ops import functional as Fn
    from verl_b200.ops.moe import _experts_grouped

    torch.manual_seed(0)
    E, H, I = 8, 512, 256
    counts = torch.tensor([300, 0, 17, 128, 129, 1, 511, 64], device="cuda")
    n = int(counts.sum())
    xp = torch.randn(n, H, device="cuda").bfloat16().requires_grad_(True)
    gu = (0.05 * torch.randn(E, 2 * I, H, device="cuda")).bfloat16().requires_grad_(True)
    dn = (0.05 * torch.randn(E, H, I, device="cuda")).bfloat16().requires_grad_(True)
    y = _experts_grouped(xp, counts, gu, dn)
    gy = torch.randn_like(y)
    gx, ggu, gdn = torch.autograd.grad(y, (xp, gu, dn), gy)
    # reference: fp32 loop over experts
    xr, gur, dnr = (t.detach().float().requires_grad_(True) for t in (xp, gu, dn))
    outs, s = [], 0
    for e, c in enumerate(counts.tolist()):
        seg = xr[s:s + c]
        g, u = (seg @ gur[e].t()).split(I, dim=-1)
        outs.append((torch.nn.functional.silu(g) * u) @ dnr[e].t())
        s += c
    ref = torch.cat(outs)
    rgx, rggu, rgdn = torch.autograd.grad(ref, (xr, gur, dnr), gy.float())
    rel = lambda a, b: ((a.float() - b).norm() / (b.norm() + 1e-9)).item()
    assert rel(y, ref) < 2e-2 and rel(gx, rgx) < 3e-2 and rel(ggu, rggu) < 3e-2 and rel(gdn, rgdn) < 3e-2, (rel(y, ref), rel(gx, rgx), rel(ggu, rggu), rel(gdn, rgdn))
    assert ggu[1].abs().sum() == 0          # an expert without tokens gets no gradient


def test_gae_scan_and_whitening_match_the_reference_loop():
    from verl_b200.ops.rl import gae_advantage
    from verl_b200.trainer.ppo import core_algos

    torch.manual_seed(0)
    B, R = 37, 300
    rewards = torch.zeros(B, R, device="cuda")
    values = torch.randn(B, R, device="cuda")
    mask = torch.ones(B, R, device="cuda")
    for i in range(B):
        n = int(torch.randint(1, R, (1,)))
        mask[i, n:] = 0
        rewards[i, n - 1] = float(torch.randn(()))
    mask[3, 10:20] = 0                                       # holes (tool outputs of a multi-turn response)
    adv, ret = gae_advantage(rewards, values, mask, 0.99, 0.95, whiten=True)
    want_adv, want_ret = core_algos.compute_gae_advantage_return(rewards.cpu(), values.cpu(), mask.cpu(), 0.99, 0.95)
    assert torch.allclose(ret.cpu(), want_ret, atol=1e-4) and torch.allclose(adv.cpu(), want_adv, atol=2e-4)
    raw, _ = gae_advantage(rewards, values, mask, 1.0, 1.0, whiten=False)
    # gamma = lambda = 1: the advantage of a token is (sum of later rewards) - its value
    i = 5
    n = int(mask[i].sum())
    assert abs(raw[i, 0].item() - (rewards[i].sum().item() - values[i, 0].item())) < 1e-4 and n > 0
    # the estimator registry takes the kernel path for CUDA tensors
    a2, r2 = core_algos.compute_gae_advantage_return(rewards, values, mask, 0.99, 0.95)
    assert torch.equal(a2, adv) and torch.equal(r2, ret)


def test_fused_value_loss_matches_autograd():
    from verl_b200.ops.rl import agg_weights, fused_value_loss
    from verl_b200.trainer.ppo import core_algos

    torch.manual_seed(1)
    B, R = 16, 200
    v = torch.randn(B, R, device="cuda", requires_grad=True)
    v_old = v.detach() + 0.6 * torch.randn(B, R, device="cuda")
    ret = torch.randn(B, R, device="cuda")
    mask = (torch.rand(B, R, device="cuda") > 0.2).float()
    for mode in ("token-mean", "seq-mean-token-mean"):
        w = agg_weights(mask, mode)
        loss, frac = fused_value_loss(v, v_old, ret, mask, w, 0.5)
        (g,) = torch.autograd.grad(loss, v)
        v2 = v.detach().clone().requires_grad_(True)
        want, want_frac = core_algos.compute_value_loss(v2, ret, v_old, mask, 0.5, mode)
        (g2,) = torch.autograd.grad(want, v2)
        assert abs(loss.item() - want.item()) < 1e-5 * max(1.0, abs(want.item())) and abs(frac.item() - want_frac.item()) < 1e-6
        assert torch.allclose(g, g2, atol=1e-7, rtol=1e-4)
