"""Ulysses sequence parallelism and context parallelism (all-gathered K/V) in the sharded-DP engine on gloo ranks: outputs
and gradients equal the single-rank run."""

import os
import subprocess
import sys

import pytest
import torch

from tests.test_engine_on_cpu import loss_fn, make_batch
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.fsdp.engine import FSDPEngine

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from tests.test_engine_on_cpu import make_batch, loss_fn
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.fsdp.engine import FSDPEngine
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
sp = int(os.environ["SP"])
key = "context_parallel_size" if os.environ.get("MODE", "").startswith("context") else "ulysses_sequence_parallel_size"
eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1, key: sp, "context_parallel_zigzag": os.environ.get("MODE") == "context_zigzag"},
                 {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
assert eng._cp_zigzag == (os.environ.get("MODE") == "context_zigzag")
eng.initialize()
assert eng.get_data_parallel_size() == world // sp
data = make_batch().chunk(eng.get_data_parallel_size())[eng.get_data_parallel_rank()]
data.meta_info["micro_batch_size_per_gpu"] = 3
lp = eng.infer_batch(data)["model_output"]["log_probs"]
eng.optimizer_zero_grad()
out = eng.forward_backward_batch(data, loss_fn)
g = eng.store.grad.clone()
dist.all_reduce(g)
g /= world
gn = eng.optimizer_step()
torch.save({"lp": lp, "ent": out["model_output"]["entropy"], "grad": g, "gn": gn, "dp_rank": eng.get_data_parallel_rank()}, os.environ["OUT"] + f".{rank}")
dist.barrier()
'''


@pytest.mark.parametrize("world,sp,mode", [(2, 2, "ulysses"), (4, 2, "ulysses"), (2, 2, "context"), (3, 3, "context"), (4, 2, "context"),
                                           (2, 2, "context_zigzag"), (3, 3, "context_zigzag"), (4, 2, "context_zigzag")])
def test_ulysses_ranks_match_single_rank(tmp_path, world, sp, mode):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    out = tmp_path / "out.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1", SP=str(sp), MODE=mode)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29750 + world + {"ulysses": 0, "context": 10, "context_zigzag": 20}[mode]), str(script)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
    eng.initialize()
    data = make_batch()
    data.meta_info["micro_batch_size_per_gpu"] = 3
    lp = eng.infer_batch(data)["model_output"]["log_probs"]
    eng.optimizer_zero_grad()
    ent = eng.forward_backward_batch(data, loss_fn)["model_output"]["entropy"]
    grad = eng.store.grad.clone()
    gn = eng.optimizer_step()
    dp = world // sp
    per = len(data) // dp
    for rk in range(world):
        res = torch.load(str(out) + f".{rk}")
        sl = slice(res["dp_rank"] * per, (res["dp_rank"] + 1) * per)
        assert torch.allclose(res["lp"], lp[sl], atol=2e-5), (res["lp"] - lp[sl]).abs().max()
        assert torch.allclose(res["ent"], ent[sl], atol=2e-5)
        n = min(grad.numel(), res["grad"].numel())
        assert torch.allclose(res["grad"][:n], grad[:n], atol=2e-6, rtol=1e-4), (res["grad"][:n] - grad[:n]).abs().max()
        assert abs(res["gn"] - gn) < 1e-4 * max(1.0, gn)
