"""Prefix sharing: one prompt forward/backward for the n responses of its group gives the same log-probs and gradients."""

import torch

from verl_b200.models.config import PRESETS
from verl_b200.protocol import DataProto
from verl_b200.utils.prefix_sharing import build_shared_pack, group_preserving_micro_batches, prompt_groups
from verl_b200.workers.engine.fsdp.engine import FSDPEngine
from verl_b200.workers.utils.losses import ppo_loss

ACTOR_CFG = {"clip_ratio": 0.2, "use_kl_loss": True, "kl_loss_coef": 1e-3, "entropy_coeff": 0.0, "loss_agg_mode": "token-mean"}


def grouped_batch(n_prompts=3, n=4, P=12, R=10, vocab=2048, seed=0, **meta):
    g = torch.Generator().manual_seed(seed)
    bs = n_prompts * n
    prompts = torch.randint(10, vocab, (n_prompts, P), generator=g)
    patt = torch.ones(n_prompts, P, dtype=torch.int64)
    for i in range(n_prompts):
        patt[i, : int(torch.randint(0, 5, (1,), generator=g))] = 0         # left padding differs per prompt
    ids = torch.cat([prompts.repeat_interleave(n, 0), torch.randint(10, vocab, (bs, R), generator=g)], 1)
    att = torch.cat([patt.repeat_interleave(n, 0), torch.ones(bs, R, dtype=torch.int64)], 1)
    for i in range(bs):
        k = int(torch.randint(0, 4, (1,), generator=g))
        if k:
            att[i, -k:] = 0
    pos = torch.clip(torch.cumsum(att, -1) - 1, min=0)
    m = {"micro_batch_size_per_gpu": bs, "temperature": 1.0, "calculate_entropy": True}
    m.update(meta)
    return DataProto.from_dict(tensors={
        "input_ids": ids, "attention_mask": att, "position_ids": pos, "responses": ids[:, -R:], "response_mask": att[:, -R:],
        "old_log_probs": -7.6 + 0.1 * torch.randn(bs, R, generator=g), "ref_log_prob": -7.6 + 0.1 * torch.randn(bs, R, generator=g),
        "advantages": torch.randn(bs, R, generator=g)}, meta_info=m)


def loss_fn(model_output, data, dp_group=None):
    return ppo_loss(ACTOR_CFG, model_output, data)


def test_pack_indices():
    data = grouped_batch()
    b = data.batch
    P = b["input_ids"].shape[1] - b["responses"].shape[1]
    gid, first = prompt_groups(b["input_ids"], b["attention_mask"], P)
    assert gid.unique().numel() == 3 and first.tolist() == [0] * 4 + [4] * 4 + [8] * 4
    sp = build_shared_pack(b["attention_mask"], P, first)
    att = b["attention_mask"].bool()
    full_ids = b["input_ids"][att]
    uniq_ids = b["input_ids"][sp.keep]
    assert sp.n_full == int(att.sum()) and sp.n_unique == int(att[:, P:].sum() + att[::4, :P].sum())
    assert torch.equal(uniq_ids[sp.expand], full_ids)          # expanding the unique tokens reproduces the packed batch
    assert torch.equal(full_ids[sp.back], uniq_ids)


def test_group_preserving_micro_batches():
    rl, pl, gid = [10] * 12, [8] * 12, [0] * 4 + [1] * 4 + [2] * 4
    parts = group_preserving_micro_batches(rl, pl, gid, max_tokens=60)
    assert sorted(i for p in parts for i in p) == list(range(12))
    for p in parts:
        groups = {gid[i] for i in p}
        assert sum(rl[i] for i in p) + 8 * len(groups) <= 60
    assert len(group_preserving_micro_batches(rl, pl, gid, max_tokens=60, num_micro_batches=len(parts) + 2)) == len(parts) + 2


def _run(meta):
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1, "dtype": "float32"}, {"lr": 1e-3}, {})
    eng.initialize()
    data = grouped_batch(**meta)
    seen, orig = [], eng.model.forward_hidden
    eng.model.forward_hidden = lambda pb, *a, **k: (seen.append(pb.input_ids.numel()), orig(pb, *a, **k))[1]
    lp = eng.infer_batch(data)["model_output"]
    full = int(data.batch["attention_mask"].sum())
    assert (sum(seen) < 0.7 * full) if meta.get("use_prefix_grouper") else (sum(seen) == full)   # the model saw each prompt once
    eng.model.forward_hidden = orig
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(data, loss_fn)
    return lp, eng.store.grad.clone()


def test_shared_prefix_matches_plain_forward_and_backward():
    lp0, g0 = _run({})
    lp1, g1 = _run({"use_prefix_grouper": True})
    assert torch.allclose(lp0["log_probs"], lp1["log_probs"], atol=2e-4), (lp0["log_probs"] - lp1["log_probs"]).abs().max()
    assert torch.allclose(lp0["entropy"], lp1["entropy"], atol=2e-4)
    assert (g0 - g1).abs().max() <= 2e-3 * g0.abs().max() + 1e-6, ((g0 - g1).abs().max(), g0.abs().max())
    # dynamic batching keeps groups together and still matches
    lp2, g2 = _run({"use_prefix_grouper": True, "use_dynamic_bsz": True, "max_token_len_per_gpu": 100})
    assert torch.allclose(lp0["log_probs"], lp2["log_probs"], atol=2e-4)
    assert (g0 - g2).abs().max() <= 2e-3 * g0.abs().max() + 1e-6


def test_trainer_step_with_prefix_sharing_and_score_centering(tmp_path):
    """End to end on CPU: the rollout engine returns the sampler's top-k head, the update pass (prefix-shared packing)
    evaluates that head under the trainer and the REINFORCE bypass loss adds the centering term."""
    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.utils.config import load_config

    ov = ["data.synthetic.enable=true", "data.synthetic.num_prompts=32", "data.train_batch_size=4", "data.max_prompt_length=32",
          "data.max_response_length=8", "actor_rollout_ref.model.preset=tiny-qwen2", "actor_rollout_ref.rollout.n=4",
          "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=16",
          "actor_rollout_ref.actor.use_kl_loss=false", "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=16",
          "actor_rollout_ref.rollout.max_num_seqs=16", "actor_rollout_ref.rollout.topk_log_probs=4",
          "actor_rollout_ref.actor.use_prefix_grouper=true", "actor_rollout_ref.model.enable_gradient_checkpointing=false",
          "algorithm.adv_estimator=grpo", "algorithm.rollout_correction.bypass_mode=true", "algorithm.rollout_correction.loss_type=reinforce",
          "algorithm.rollout_correction.rollout_is=token", "algorithm.rollout_correction.score_centering=true",
          "reward.reward_manager=token_rule", "trainer.device=cpu", "trainer.val_before_train=false", "trainer.logger=[]",
          "trainer.n_gpus_per_node=1", "data.shuffle=false", f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.total_training_steps=1"]
    cfg = load_config("ppo_trainer", ov)
    tr = PPOTrainer(cfg, reward_fn=load_reward_manager(cfg, None), val_reward_fn=None)
    tr.init_workers()
    tr.global_steps = 1
    m = tr.step(next(iter(tr.train_dataloader)))
    b = tr._last_batch.batch
    assert b["rollout_topk_ids"].shape == (16, 8, 4)
    # the sampled token's log-prob can never exceed the best head entry; head entries are sorted
    lps, top = b["rollout_log_probs"], b["rollout_topk_log_probs"]
    mask = b["response_mask"].bool()
    assert (lps[mask] <= top[..., 0][mask] + 1e-5).all() and (top[..., 0] >= top[..., 1]).all()
    for k in ("actor/sc_correction", "actor/sc_sampler_head_mass", "actor/sc_train_head_mass", "actor/grad_norm"):
        assert k in m, (k, sorted(m))
    # same weights on both sides in the first step: the trainer's head mass equals the sampler's
    assert abs(m["actor/sc_sampler_head_mass"] - m["actor/sc_train_head_mass"]) < 1e-4


def test_on_policy_distillation_step(tmp_path):
    """A frozen teacher (same architecture, other weights) scores the student's samples; the actor's loss is the forward KL to
    the teacher's top-k head and a few steps reduce it."""
    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.utils.config import load_config

    ov = ["data.synthetic.enable=true", "data.synthetic.num_prompts=64", "data.train_batch_size=4", "data.max_prompt_length=32",
          "data.max_response_length=8", "actor_rollout_ref.model.preset=tiny-qwen2", "actor_rollout_ref.rollout.n=2",
          "actor_rollout_ref.actor.ppo_mini_batch_size=2", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
          "actor_rollout_ref.actor.use_kl_loss=false", "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8",
          "actor_rollout_ref.rollout.max_num_seqs=8", "actor_rollout_ref.model.enable_gradient_checkpointing=false",
          "actor_rollout_ref.actor.optim.lr=3e-3", "actor_rollout_ref.distillation.enable=true", "actor_rollout_ref.distillation.teacher_model.preset=tiny-qwen2",
          "actor_rollout_ref.distillation.topk=8", "+actor_rollout_ref.ref.fsdp_config.seed=7", "+actor_rollout_ref.actor.fsdp_config.seed=1",
          "algorithm.adv_estimator=grpo", "reward.reward_manager=token_rule", "trainer.device=cpu", "trainer.val_before_train=false",
          "trainer.logger=[]", "trainer.n_gpus_per_node=1", "data.shuffle=false", f"trainer.default_local_dir={tmp_path}/ckpt",
          "trainer.total_training_steps=4"]
    cfg = load_config("ppo_trainer", ov)
    tr = PPOTrainer(cfg, reward_fn=load_reward_manager(cfg, None), val_reward_fn=None)
    tr.init_workers()
    w = tr.actor_rollout_wg.worker
    assert w.teacher is not None and not torch.equal(w.teacher.engine.store.flat, w.actor.engine.store.flat)   # a different model
    it = iter(tr.train_dataloader)
    losses = []
    for step in range(1, 5):
        tr.global_steps = step
        m = tr.step(next(it))
        losses.append(m["distill/forward_kl"])
        assert "timing_s/teacher" in m and 0.0 <= m["distill/top1_agreement"] <= 1.0
    b = tr._last_batch.batch
    assert b["teacher_topk_ids"].shape == (8, 8, 8) and (b["teacher_topk_log_probs"][..., 0] >= b["teacher_topk_log_probs"][..., 1]).all()
    assert losses[0] > 0 and min(losses[1:]) < losses[0], losses
