"""GRPO plumbing configuration end to end on CPU: tiny Qwen2-arch model, synthetic prompts, mod-7 rule reward."""

import json
import os
import subprocess
import sys

import pytest
import torch

from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer, apply_kl_penalty, compute_advantage
from verl_b200.trainer.ppo.reward import load_reward_manager
from verl_b200.utils.config import load_config

OV = ["data.synthetic.enable=true", "data.synthetic.num_prompts=64", "data.train_batch_size=8", "data.max_prompt_length=32",
      "data.max_response_length=16", "actor_rollout_ref.model.preset=tiny-qwen2", "actor_rollout_ref.rollout.n=4",
      "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
      "actor_rollout_ref.actor.use_kl_loss=true", "actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=16",
      "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=16", "actor_rollout_ref.rollout.max_num_seqs=32",
      "actor_rollout_ref.model.enable_gradient_checkpointing=false", "algorithm.adv_estimator=grpo", "reward.reward_manager=token_rule",
      "trainer.device=cpu", "trainer.val_before_train=false", "trainer.logger=[]", "trainer.n_gpus_per_node=1", "data.shuffle=false"]


def build(tmp_path, extra=()):
    cfg = load_config("ppo_trainer", OV + [f"trainer.default_local_dir={tmp_path}/ckpt"] + list(extra))
    tr = PPOTrainer(cfg, reward_fn=load_reward_manager(cfg, None), val_reward_fn=load_reward_manager(cfg, None))
    tr.init_workers()
    return tr


def test_grpo_steps_and_metric_names(tmp_path):
    tr = build(tmp_path, ["trainer.total_training_steps=2"])
    it = iter(tr.train_dataloader)
    tr.global_steps = 1
    m = tr.step(next(it))
    for k in ["actor/pg_loss", "actor/pg_clipfrac", "actor/ppo_kl", "actor/kl_loss", "actor/grad_norm", "actor/lr", "actor/entropy",
              "critic/score/mean", "critic/rewards/mean", "critic/advantages/mean", "response_length/mean", "prompt_length/mean",
              "timing_s/gen", "timing_s/old_log_prob", "timing_s/ref", "timing_s/update_actor", "timing_s/update_weights", "timing_s/step",
              "perf/total_num_tokens", "perf/time_per_step", "perf/throughput", "perf/mfu/actor"]:
        assert k in m, k
    # on-policy first mini-batch: ratio 1, and the rollout engine's log-probs equal the trainer's recomputation (fp32)
    assert abs(m["actor/ppo_kl"]) < 1e-4 and m["training/rollout_probs_diff_max"] < 1e-5
    b = tr._last_batch.batch
    assert b["responses"].shape == (32, 16) and (b["token_level_scores"].sum(-1) <= 1).all()
    uid = tr._last_batch.non_tensor_batch["uid"]
    adv = b["advantages"]
    for u in set(uid.tolist()):           # group-normalised: mean zero within each prompt group
        rows = [i for i, x in enumerate(uid) if x == u]
        assert len(rows) == 4
        assert abs(sum(adv[i, 0].item() for i in rows)) < 1e-4


def test_fit_saves_and_resumes(tmp_path):
    tr = build(tmp_path, ["trainer.total_training_steps=2", "trainer.save_freq=1", "trainer.resume_mode=auto"])
    tr.fit()
    root = tmp_path / "ckpt"
    assert (root / "latest_checkpointed_iteration.txt").read_text() == "2"
    assert (root / "global_step_2" / "actor" / "model_world_size_1_rank_0.pt").exists() and (root / "global_step_2" / "data.pt").exists()
    flat = tr.actor_rollout_wg.worker.actor.engine.store.flat.clone()
    tr2 = build(tmp_path, ["trainer.total_training_steps=3", "trainer.save_freq=-1", "trainer.resume_mode=auto"])
    assert tr2._load_checkpoint() == 2
    assert torch.equal(tr2.actor_rollout_wg.worker.actor.engine.store.flat, flat)
    # a corrupted tracker file falls back to training from scratch instead of crashing
    (root / "latest_checkpointed_iteration.txt").write_text("not-a-number")
    tr3 = build(tmp_path, ["trainer.resume_mode=auto"])
    assert tr3._load_checkpoint() == 0


def test_gae_with_critic_runs(tmp_path):
    tr = build(tmp_path, ["algorithm.adv_estimator=gae", "critic.model.preset=tiny-qwen2", "critic.ppo_micro_batch_size_per_gpu=8",
                          "critic.model.enable_gradient_checkpointing=false", "actor_rollout_ref.rollout.n=1", "actor_rollout_ref.actor.use_kl_loss=false",
                          "algorithm.use_kl_in_reward=true", "trainer.total_training_steps=1"])
    tr.global_steps = 1
    m = tr.step(next(iter(tr.train_dataloader)))
    assert "critic/vf_loss" in m and "critic/values/mean" in m and "actor/reward_kl_penalty" in m and "critic/grad_norm" in m


@pytest.mark.parametrize("zero3", [False, True])
def test_two_rank_gloo_fit(tmp_path, zero3):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    logf = tmp_path / "log.jsonl"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29671",
           "-m", "verl_b200.trainer.main_ppo"] + [o for o in OV if not o.startswith("trainer.logger")] + \
          ["trainer.logger=[file]", "trainer.total_training_steps=2", f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.resume_mode=disable"]
    if zero3:      # row-sharded projections in actor and reference; the rollout keeps its own gathered copy
        cmd += ["actor_rollout_ref.actor.fsdp_config.reshard_after_forward=true", "+actor_rollout_ref.ref.fsdp_config.reshard_after_forward=true",
                "trainer.save_freq=2"]
    env = dict(os.environ, VERL_FILE_LOGGER_PATH=str(logf), OMP_NUM_THREADS="2", PYTHONPATH=repo)
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=repo)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rows = [json.loads(x) for x in logf.read_text().splitlines()]
    assert len(rows) == 2 and rows[-1]["data"]["perf/total_num_tokens"] > 0 and abs(rows[0]["data"]["actor/ppo_kl"]) < 1e-4
    if zero3:
        assert os.path.exists(tmp_path / "ckpt" / "global_step_2" / "actor" / "model_world_size_2_rank_1.pt")


def test_reward_model_worker_scores_the_last_response_token(tmp_path):
    """A frozen scalar-head model scores every trajectory; its score lands on the last response token and is added to the rule
    reward before advantages are computed."""
    tr = build(tmp_path, ["trainer.total_training_steps=1", "reward.reward_model.enable=true", "reward.reward_model.preset=tiny-qwen2",
                          "reward.reward_model.micro_batch_size_per_gpu=16"])
    assert tr.rm_wg is not None and tr.rm_wg.worker.rm.engine.cfg.value_head and tr.rm_wg.worker.rm.engine.forward_only
    tr.global_steps = 1
    m = tr.step(next(iter(tr.train_dataloader)))
    assert "reward_model/score_mean" in m
    b = tr._last_batch.batch
    rm = tr.rm_wg.compute_rm_score(tr._last_batch).batch["rm_scores"]
    mask = b["response_mask"]
    last = (mask.sum(-1) - 1).long()
    rows = torch.arange(rm.shape[0])
    assert (rm.abs().sum(-1) == rm[rows, last].abs()).all() and rm[rows, last].abs().sum() > 0       # one non-zero entry per row, at the last token
    rule = b["token_level_scores"] - rm
    assert ((rule == 0) | (rule == 1)).all()                                                            # what is left is the 0/1 rule reward


def test_rollout_dumps_and_viewer(tmp_path, capsys):
    """``trainer.rollout_data_dir``: one JSON line per trajectory and step; the viewer lists, filters and summarises them."""
    from verl_b200.scripts.rollout_viewer import list_steps, load_step, main as viewer_main

    dump = tmp_path / "rollouts"
    tr = build(tmp_path, ["trainer.total_training_steps=2", f"trainer.rollout_data_dir={dump}"])
    it = iter(tr.train_dataloader)
    for step in (1, 2):
        tr.global_steps = step
        tr.step(next(it))
    assert list_steps(str(dump)) == [1, 2]
    rows = load_step(str(dump), 2)
    assert len(rows) == 8 * 4 and {"input", "output", "score", "step"} <= set(rows[0]) and rows[0]["step"] == 2
    assert viewer_main([str(dump), "--stats"]) == 0
    out = capsys.readouterr().out
    assert "mean score" in out and out.strip().splitlines()[-1].split()[0] == "2"
    assert viewer_main([str(dump), "--step", "1", "--sort=-score", "--limit", "3"]) == 0
    out = capsys.readouterr().out
    assert out.count("--- output") == 3 and "step 1: 32 trajectories" in out


def test_mini_batch_counts_prompts_not_trajectories(tmp_path):
    """``ppo_mini_batch_size`` is a number of prompts: 8 prompts x n=4 with a mini-batch of 4 prompts is two optimizer steps
    per RL step (not eight), and a mini-batch equal to the train batch is exactly one."""
    for mini, want in ((4, 2), (8, 1)):
        tr = build(tmp_path, ["trainer.total_training_steps=1", f"actor_rollout_ref.actor.ppo_mini_batch_size={mini}"])
        eng = tr.actor_rollout_wg.worker.actor.engine
        before = eng.step_count
        tr.global_steps = 1
        tr.step(next(iter(tr.train_dataloader)))
        assert eng.step_count - before == want


def test_model_only_resume_continues_from_the_loaded_weights(tmp_path):
    """Checkpoint without optimizer state: after the load the fp32 master copy must equal the loaded weights, so the next
    optimizer step moves the LOADED weights instead of writing the initialisation-time master over them."""
    ck = ["actor_rollout_ref.actor.checkpoint.save_contents=[model,extra]", "actor_rollout_ref.actor.checkpoint.load_contents=[model,extra]",
          "actor_rollout_ref.actor.optim.lr=1e-3"]
    tr = build(tmp_path, ["trainer.total_training_steps=3", "trainer.save_freq=-1"] + ck)
    it = iter(tr.train_dataloader)
    tr.global_steps = 1
    tr.step(next(it))
    tr._save_checkpoint()
    eng = tr.actor_rollout_wg.worker.actor.engine
    saved = eng.store.flat.clone()
    assert not os.path.exists(tmp_path / "ckpt" / "global_step_1" / "actor" / "optim_world_size_1_rank_0.pt")
    tr2 = build(tmp_path, ["trainer.total_training_steps=3", "trainer.resume_mode=auto"] + ck)
    eng2 = tr2.actor_rollout_wg.worker.actor.engine
    init = eng2.store.flat.clone()
    assert tr2._load_checkpoint() == 1
    assert torch.equal(eng2.store.flat, saved) and not torch.equal(saved, init)
    assert torch.equal(eng2.master, saved[eng2.store.shard_slice].float())
    assert float(eng2.exp_avg.abs().sum()) == 0.0 and eng2.step_count == 0
    tr2.global_steps = 2
    tr2.step(next(iter(tr2.train_dataloader)))
    after = eng2.store.flat
    # one AdamW step at lr 1e-3 moves every weight by at most about lr from where it was loaded
    assert float((after.float() - saved.float()).abs().max()) < 5e-3
    assert float((after.float() - init.float()).abs().max()) > 5e-3 or float((saved.float() - init.float()).abs().max()) < 5e-3


def test_async_save_names_a_step_only_when_all_writers_finished(tmp_path):
    """Asynchronous saves: the tracker file appears after the background writer has dropped its marker, and pruning keeps
    the last complete checkpoint while a newer one is still being written."""
    tr = build(tmp_path, ["trainer.total_training_steps=3", "trainer.save_freq=1", "trainer.max_actor_ckpt_to_keep=1",
                          "actor_rollout_ref.actor.checkpoint.async_save=true"])
    tr.fit()
    root = tmp_path / "ckpt"
    assert (root / "latest_checkpointed_iteration.txt").read_text() == "3"
    last = root / "global_step_3" / "actor"
    assert (last / "model_world_size_1_rank_0.pt").exists() and not (last / ".async_save_pending").exists()
    assert not [f for f in os.listdir(last) if f.startswith(".async_done")]
    kept = sorted(d for d in os.listdir(root) if d.startswith("global_step_") and os.path.exists(root / d / "actor" / "model_world_size_1_rank_0.pt"))
    assert "global_step_3" in kept and "global_step_1" not in kept


@pytest.mark.parametrize("mode", ["R3", "R2"])
def test_router_replay_end_to_end(tmp_path, mode):
    """Mixture-of-experts actor with router replay. R3: the rollout engine records the experts of every token, the
    old-log-prob pass and the update replay them. R2: the old-log-prob pass records, the update replays. Either way the
    batch carries ``routed_experts`` [bs, prompt + response, layers, topk] and the first mini-batch is exactly on-policy."""
    extra = ["trainer.total_training_steps=1", "actor_rollout_ref.model.preset=tiny-qwen3-moe", f"actor_rollout_ref.actor.router_replay.mode={mode}",
             "actor_rollout_ref.actor.use_kl_loss=false"]
    if mode == "R3":
        extra.append("actor_rollout_ref.rollout.enable_rollout_routing_replay=true")
    tr = build(tmp_path, extra)
    tr.global_steps = 1
    m = tr.step(next(iter(tr.train_dataloader)))
    b = tr._last_batch.batch
    assert "routed_experts" in b.keys()
    rt = b["routed_experts"]
    assert rt.shape[:2] == b["input_ids"].shape and rt.shape[2:] == (2, 2)
    att = b["attention_mask"].bool()
    assert int(rt[att].min()) >= 0 and int(rt[att].max()) < 8 and bool((rt[~att] == -1).all())
    assert abs(m["actor/ppo_kl"]) < 1e-4
    if mode == "R3":
        assert m["training/rollout_probs_diff_max"] < 1e-4


def test_fit_brackets_the_listed_steps_with_the_worker_profilers(tmp_path):
    """``global_profiler.steps`` + a role's ``profiler.enable``: the trainer starts the workers' profilers before a listed step and
    stops them after it (one capture for consecutive steps with ``profile_continuous_steps``); the torch tool writes a trace per
    capture, and the worker entry points run inside named ranges."""
    prof_dir = tmp_path / "prof"
    tr = build(tmp_path, ["trainer.total_training_steps=4", "global_profiler.tool=torch", "global_profiler.steps=[2,3]",
                          "global_profiler.profile_continuous_steps=true", f"global_profiler.save_path={prof_dir}",
                          "actor_rollout_ref.actor.profiler.enable=true", "actor_rollout_ref.actor.profiler.all_ranks=true"])
    w = tr.actor_rollout_wg.worker
    assert w.profiler.enabled and w.profiler.config.tool == "torch" and w.profiler.config.save_path == str(prof_dir)
    calls = []
    start, stop = w.profiler.start, w.profiler.stop
    w.profiler.start = lambda **kw: (calls.append(("start", tr.global_steps, kw.get("profile_step"))), start(**kw))[1]
    w.profiler.stop = lambda: (calls.append(("stop", tr.global_steps)), stop())[1]
    tr.fit()
    assert calls == [("start", 2, 2), ("stop", 3)]                     # steps 2 and 3 share one capture
    assert any(f.endswith(".json") or f.endswith(".json.gz") for _, _, fs in os.walk(prof_dir) for f in fs), list(os.walk(prof_dir))
    # a role without profiler.enable stays off, and the facade is a no-op for it
    tr2 = build(tmp_path, ["trainer.total_training_steps=1", "global_profiler.tool=torch", "global_profiler.steps=[1]"])
    assert not tr2.actor_rollout_wg.worker.profiler.enabled
    tr2.fit()
