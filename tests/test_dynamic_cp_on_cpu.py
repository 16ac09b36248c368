"""Dynamic context parallelism: per-sample group sizes, aligned rank groups, packing under the per-rank token cap."""

import pytest
import torch

from verl_b200.utils.dynamic_cp_scheduler import DynamicCPScheduler, cp_members, local_padding_mask, postprocess_dynamic_cp_batch


def _check(sched, seq_lens, mbs):
    R, cap = sched.total_ranks, sched.max_seqlen_per_dp_cp_rank
    seen = []
    for assign in mbs:
        assert len(assign) == R
        groups = {}
        for r, ids in enumerate(assign):
            if ids:
                groups.setdefault(tuple(ids), []).append(r)
        for ids, ranks in groups.items():
            k = len(ranks)
            assert ranks == list(range(ranks[0], ranks[0] + k)) and k & (k - 1) == 0 and ranks[0] % k == 0      # aligned power of two
            assert sum(seq_lens[i] for i in ids) / k <= cap                                                # per-rank share under the cap
            seen += list(ids)
    assert sorted(seen) == list(range(len(seq_lens)))                                                     # every sample exactly once


def test_short_samples_stay_on_one_rank_and_long_ones_span_aligned_groups():
    s = DynamicCPScheduler(max_seqlen_per_dp_cp_rank=1000, dp_size=2, cp_size=4)
    lens = [3500, 900, 800, 1900, 120, 100, 90, 2500, 700]
    mbs = s.schedule_lengths(lens)
    _check(s, lens, mbs)
    first = mbs[0]
    assert len(cp_members(first, next(r for r, ids in enumerate(first) if 0 in ids))) == 4                # 3500 tokens need 4 ranks
    assert s.ranks_needed(900) == 1 and s.ranks_needed(1900) == 2 and s.ranks_needed(2500) == 4
    with pytest.raises(ValueError):
        s.schedule_lengths([9000])                                                                       # needs 16 ranks, 8 exist
    with pytest.raises(ValueError):
        s.schedule_lengths([])


def test_idle_ranks_are_absorbed_or_fed():
    s = DynamicCPScheduler(max_seqlen_per_dp_cp_rank=1000, dp_size=1, cp_size=8)
    mbs = s.schedule_lengths([500])                                      # one short sample on eight ranks: the group grows to all of them
    assert len(mbs) == 1 and all(ids == [0] for ids in mbs[0])
    lens = [400, 300, 200]
    mbs = s.schedule_lengths(lens)                                      # three samples share one rank at first; idle ranks take samples over
    _check(s, lens, mbs)
    assert len(mbs) == 1 and sum(1 for ids in mbs[0] if ids) == 8
    g = torch.Generator().manual_seed(0)
    for _ in range(20):
        lens = torch.randint(1, 7000, (int(torch.randint(1, 40, (1,), generator=g)),), generator=g).tolist()
        _check(s, lens, s.schedule_lengths(lens))


def test_rank_view_padding_mask_and_collection():
    s = DynamicCPScheduler(max_seqlen_per_dp_cp_rank=64, dp_size=1, cp_size=4)
    lens = [100, 30, 20, 10]
    views = [s.schedule(lens, r, tp_size=1, cp_layout="zigzag") for r in range(4)]
    n_mb = len(views[0])
    assert all(len(v) == n_mb for v in views)
    outs = [[] for _ in range(4)]
    for j in range(n_mb):
        for r in range(4):
            mb = views[r][j]
            if not mb["sample_ids"]:
                continue
            k = mb["local_cp_size"]
            # the shards of a group cover every real token exactly once
            if mb["group_leader"]:
                total = sum(views[m][j]["local_num_tokens"] for m in mb["members"])
                assert total == sum(lens[i] for i in mb["sample_ids"])
            assert mb["padding_mask"].numel() * k == sum(-(-lens[i] // (2 * k if k > 1 else 1)) * (2 * k if k > 1 else 1) for i in mb["sample_ids"])
            outs[r].append({"group_leader": mb["group_leader"], "sample_ids": mb["sample_ids"], "loss": float(r),
                            "metrics": {"m": [1.0]}, "model_output": {"log_probs": [torch.full((lens[i],), float(i)) for i in mb["sample_ids"]]}})
    merged = postprocess_dynamic_cp_batch([o for r in range(4) for o in outs[r]], len(lens))
    assert [int(t[0]) for t in merged["model_output"]["log_probs"]] == [0, 1, 2, 3]
    assert [t.numel() for t in merged["model_output"]["log_probs"]] == lens
    # contiguous layout: the mask marks the tail padding of the sequence that crosses into this rank's slice
    m = local_padding_mask([10, 5], cp_size=2, cp_rank=1, tp_size=1, cp_layout="contiguous")
    assert m.tolist() == [False] * 2 + [False] * 5 + [True]          # rows 8..15 of [10 real | 5 real + 1 pad]


import os
import subprocess
import sys

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from tests.test_dynamic_cp_on_cpu import ragged_batch
from tests.test_engine_on_cpu import loss_fn
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.fsdp.engine import FSDPEngine
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cp = int(os.environ["CP"])
eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1, "context_parallel_size": cp, "dynamic_context_parallel": True, "max_seqlen_per_dp_cp_rank": 24,
                                         "context_parallel_zigzag": os.environ["ZIGZAG"] == "1"},
                 {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
eng.initialize()
data = ragged_batch().chunk(eng.get_data_parallel_size())[eng.get_data_parallel_rank()]
lp = eng.infer_batch(data)["model_output"]["log_probs"]
eng.optimizer_zero_grad()
out = eng.forward_backward_batch(data, loss_fn)
sizes = sorted(set(eng.dcp_stats["group_sizes"]))
g = eng.store.grad.clone()
dist.all_reduce(g)
g /= world
gn = eng.optimizer_step()
torch.save({"lp": lp, "ent": out["model_output"]["entropy"], "grad": g, "gn": gn, "dp_rank": eng.get_data_parallel_rank(), "sizes": sizes,
            "n_loss": len(out["loss"]), "pg": out["metrics"]["actor/pg_loss"].values}, os.environ["OUT"] + f".{rank}")
dist.barrier()
'''


def ragged_batch():
    """Sequences of 8 to 58 tokens (left padding of very different widths) so that the scheduler uses groups of 1, 2 and 4."""
    from tests.test_engine_on_cpu import make_batch

    data = make_batch(bs=8, P=48, R=10)
    att = data.batch["attention_mask"]
    for i, cut in enumerate([0, 40, 44, 10, 30, 46, 5, 38]):
        att[i, :cut] = 0
    data.batch["position_ids"] = torch.clip(torch.cumsum(att, -1) - 1, min=0)
    return data


@pytest.mark.parametrize("world,cp,zigzag", [(4, 4, False), (4, 4, True), (4, 2, False)])
def test_dynamic_cp_ranks_match_single_rank(tmp_path, world, cp, zigzag):
    from tests.test_engine_on_cpu import loss_fn
    from verl_b200.models.config import PRESETS
    from verl_b200.workers.engine.fsdp.engine import FSDPEngine

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    out = tmp_path / "out.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1", CP=str(cp), ZIGZAG="1" if zigzag else "0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29790 + cp + (1 if zigzag else 0)), str(script)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
    eng.initialize()
    data = ragged_batch()
    data.meta_info["micro_batch_size_per_gpu"] = 4
    lp = eng.infer_batch(data)["model_output"]["log_probs"]
    eng.optimizer_zero_grad()
    ent = eng.forward_backward_batch(data, loss_fn)["model_output"]["entropy"]
    grad = eng.store.grad.clone()
    gn = eng.optimizer_step()
    dp = world // cp
    per = len(data) // dp
    sizes = set()
    for rk in range(world):
        res = torch.load(str(out) + f".{rk}")
        sl = slice(res["dp_rank"] * per, (res["dp_rank"] + 1) * per)
        assert torch.allclose(res["lp"], lp[sl], atol=2e-5), (res["lp"] - lp[sl]).abs().max()
        assert torch.allclose(res["ent"], ent[sl], atol=2e-5)
        n = min(grad.numel(), res["grad"].numel())
        assert torch.allclose(res["grad"][:n], grad[:n], atol=2e-6, rtol=1e-4), (res["grad"][:n] - grad[:n]).abs().max()
        assert abs(res["gn"] - gn) < 1e-4 * max(1.0, gn)
        sizes |= set(res["sizes"])
        # every rank of a CP group reports the same merged losses / metrics (one entry per sub-group and micro-batch)
        assert res["n_loss"] == len(res["pg"]) and res["n_loss"] >= 2
    assert len(sizes) >= 2, sizes                                    # groups of different widths were really used
