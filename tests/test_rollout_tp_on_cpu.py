"""Tensor-parallel rollout replicas on gloo ranks: lockstep generation equals the single-rank engine; GRPO end to end."""

import json
import os
import subprocess
import sys

import pytest
import torch

from verl_b200.models.config import PRESETS
from verl_b200.models.transformer import DecoderLM
from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from verl_b200.models.config import PRESETS
from verl_b200.models.parallel_model import build_rollout_shard
from verl_b200.models.transformer import DecoderLM
from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
full = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=3)
local = build_rollout_shard(full, rank, world)
assert local.layers[0].mlp.down_proj.shape[1] == full.layers[0].mlp.down_proj.shape[1] // world and local.embed_tokens is full.embed_tokens
eng = InferenceEngine(local, max_num_seqs=8, max_model_len=128, num_blocks=32, tp_group=dist.group.WORLD)
g = torch.Generator().manual_seed(0)
prompts = [torch.randint(10, 2000, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g).tolist() for _ in range(6)]
out = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
out2 = eng.generate(prompts[:3], SamplingParams(temperature=1.0, max_tokens=10, seed=5))
torch.save({"greedy": [o.token_ids for o in out], "lp": [o.log_probs for o in out], "sampled": [o.token_ids for o in out2]}, os.environ["OUT"] + f".{rank}")
dist.barrier()
'''


def test_tp2_engine_matches_tp1(tmp_path):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    out = tmp_path / "o.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29771", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    a, b = torch.load(str(out) + ".0"), torch.load(str(out) + ".1")
    assert a["greedy"] == b["greedy"] and a["sampled"] == b["sampled"]          # lockstep
    full = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=3)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(10, 2000, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g).tolist() for _ in range(6)]
    want = InferenceEngine(full, max_num_seqs=8, max_model_len=128, num_blocks=32).generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    for w, got, lp in zip(want, a["greedy"], a["lp"]):
        assert w.token_ids == got and torch.allclose(torch.tensor(w.log_probs), torch.tensor(lp), atol=1e-4)


@pytest.mark.parametrize("world", [2, 4])
def test_grpo_fit_with_tp2_rollout(tmp_path, world):
    """world = 4: two tensor-parallel replicas of two ranks each next to four data-parallel trainer ranks."""
    from tests.test_trainer_e2e_on_cpu import OV

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    logf = tmp_path / "log.jsonl"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(29771 + world),
           "-m", "verl_b200.trainer.main_ppo"] + [o for o in OV if not o.startswith("trainer.logger")] + \
          ["trainer.logger=[file]", "trainer.total_training_steps=2", f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.resume_mode=disable",
           "actor_rollout_ref.rollout.tensor_model_parallel_size=2"]
    env = dict(os.environ, VERL_FILE_LOGGER_PATH=str(logf), OMP_NUM_THREADS="2", PYTHONPATH=repo)
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=repo)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 2 and rows[-1]["perf/total_num_tokens"] > 0 and abs(rows[0]["actor/ppo_kl"]) < 1e-4
    # the rollout's log-probs and the trainer's recomputation agree: the sharded replica serves the trainer's weights
    assert abs(rows[1].get("training/rollout_probs_diff_mean", 0.0)) < 1e-3


def test_resume_hands_the_restored_weights_to_the_tp_rollout(tmp_path):
    """Tensor-parallel replicas hold their own slices of the weights. After a resume those slices must be refreshed from the
    restored weights before the first rollout: the rollout's log-probs then equal the trainer's recomputation on the very
    first resumed step (with stale slices they differ, because training moved the weights before the save)."""
    from tests.test_trainer_e2e_on_cpu import OV

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29781",
            "-m", "verl_b200.trainer.main_ppo"] + [o for o in OV if not o.startswith("trainer.logger")] + \
           ["trainer.logger=[file]", f"trainer.default_local_dir={tmp_path}/ckpt", "actor_rollout_ref.rollout.tensor_model_parallel_size=2",
            "actor_rollout_ref.actor.optim.lr=3e-3"]        # a large step, so that stale rollout weights would be visible
    log1, log2 = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    env = dict(os.environ, OMP_NUM_THREADS="2", PYTHONPATH=repo)
    r = subprocess.run(base + ["trainer.total_training_steps=2", "trainer.save_freq=2", "trainer.resume_mode=disable"],
                       env=dict(env, VERL_FILE_LOGGER_PATH=str(log1)), capture_output=True, text=True, timeout=900, cwd=repo)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text() == "2"
    r = subprocess.run(base + ["trainer.total_training_steps=3", "trainer.save_freq=-1", "trainer.resume_mode=auto"],
                       env=dict(env, VERL_FILE_LOGGER_PATH=str(log2)), capture_output=True, text=True, timeout=900, cwd=repo)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rows = [json.loads(x) for x in log2.read_text().splitlines()]
    assert len(rows) == 1 and rows[0]["step"] == 3
    assert abs(rows[0]["data"]["training/rollout_probs_diff_max"]) < 1e-4
    # the same quantity in the first run's second step shows what training did to the weights: non-trivial policy movement
    first = [json.loads(x)["data"] for x in log1.read_text().splitlines()]
    assert abs(first[1]["training/rollout_probs_diff_max"]) < 1e-4


def test_zero3_trainer_feeds_tp2_rollout_slices(tmp_path):
    """Row-sharded trainer weights (ZeRO-3 mode) → tensor-parallel rollout slices: every rank fills its slice block by block
    from the row shards (on CPU ranks through the gathered weight, on GPUs by peer-read kernels). The rollout's log-probs
    must agree with the trainer's recomputation on every step, i.e. also after the weights moved."""
    from tests.test_trainer_e2e_on_cpu import OV

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    logf = tmp_path / "log.jsonl"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29791",
           "-m", "verl_b200.trainer.main_ppo"] + [o for o in OV if not o.startswith("trainer.logger")] + \
          ["trainer.logger=[file]", "trainer.total_training_steps=3", f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.resume_mode=disable",
           "actor_rollout_ref.rollout.tensor_model_parallel_size=2", "actor_rollout_ref.actor.optim.lr=3e-3",
           "actor_rollout_ref.actor.fsdp_config.reshard_after_forward=true", "+actor_rollout_ref.ref.fsdp_config.reshard_after_forward=true"]
    env = dict(os.environ, VERL_FILE_LOGGER_PATH=str(logf), OMP_NUM_THREADS="2", PYTHONPATH=repo)
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=repo)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rows = [json.loads(x)["data"] for x in logf.read_text().splitlines()]
    assert len(rows) == 3
    for row in rows:
        assert abs(row["training/rollout_probs_diff_max"]) < 1e-4


VL_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from verl_b200.models.config import PRESETS
from verl_b200.models.parallel_model import VisionLanguageRolloutShard
from verl_b200.models.vision import VisionLanguageModel
from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
full = VisionLanguageModel(PRESETS["tiny-qwen2-vl"], dtype=torch.float32, device=torch.device("cpu"), seed=11).eval()
local = VisionLanguageRolloutShard(full, rank, world)
assert local.visual is full.visual and local.language_model.layers[0].mlp.down_proj.shape[1] == full.language_model.layers[0].mlp.down_proj.shape[1] // world
eng = InferenceEngine(local, max_num_seqs=8, max_model_len=64, num_blocks=32, tp_group=dist.group.WORLD, enforce_eager=True)
g = torch.Generator().manual_seed(2)
v = full.vcfg
prompt = [7, 8, v.vision_start_token_id] + [v.image_token_id] * 4 + [9, 10, 11]
mm = {"pixel_values": torch.randn(16, v.patch_dim, generator=g), "image_grid_thw": torch.tensor([[1, 4, 4]])}
out = eng.generate([prompt, [5, 6, 7, 8]], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), multi_modal=[mm, None])
torch.save([o.token_ids for o in out], os.environ["OUT"] + f".{rank}")
dist.barrier()
'''


def test_tp2_replica_serves_a_vision_language_model(tmp_path):
    """The decoder is cut over the replica's ranks, the vision tower runs whole on each of them: image prompts decode to the same
    tokens as on a single-rank engine."""
    from verl_b200.models.vision import VisionLanguageModel

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "vl.py"
    script.write_text(VL_WORKER)
    out = tmp_path / "vl.pt"
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29775", str(script)], env=dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1"),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    a, b = torch.load(str(out) + ".0"), torch.load(str(out) + ".1")
    assert a == b
    full = VisionLanguageModel(PRESETS["tiny-qwen2-vl"], dtype=torch.float32, device=torch.device("cpu"), seed=11).eval()
    g = torch.Generator().manual_seed(2)
    v = full.vcfg
    prompt = [7, 8, v.vision_start_token_id] + [v.image_token_id] * 4 + [9, 10, 11]
    mm = {"pixel_values": torch.randn(16, v.patch_dim, generator=g), "image_grid_thw": torch.tensor([[1, 4, 4]])}
    want = InferenceEngine(full, max_num_seqs=8, max_model_len=64, num_blocks=32, enforce_eager=True).generate(
        [prompt, [5, 6, 7, 8]], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), multi_modal=[mm, None])
    assert [list(o.token_ids) for o in want] == [list(x) for x in a]
