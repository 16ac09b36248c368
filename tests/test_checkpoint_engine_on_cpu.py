"""Weight-sync backends on gloo ranks and the quantisation reference formulas on CPU."""

import os
import subprocess
import sys

import torch

from verl_b200.checkpoint_engine import CheckpointEngineRegistry, delta_apply, delta_compact, tensor_checksum
from verl_b200.ops.quant import blockwise_cast_to_fp8, dequant_blockwise_fp8, fp4_fake_quant, fp4_fake_quant_ste, QATLinear

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from verl_b200.checkpoint_engine import CheckpointEngineRegistry
from verl_b200.models.config import PRESETS
from verl_b200.models.transformer import DecoderLM
dist.init_process_group("gloo")
rank = dist.get_rank()
backend = os.environ["BACKEND"]
eng = CheckpointEngineRegistry.new(backend, bucket_megabytes=1, dense_threshold=0.25)
src = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.bfloat16, seed=1)
dst = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.bfloat16, seed=2)
stats = []
for step in range(3):
    if step:   # a small, sparse update like a low-learning-rate RL step
        with torch.no_grad():
            g = torch.Generator().manual_seed(step)
            for p in src.parameters():
                mask = torch.rand(p.shape, generator=g) < 0.02
                p.add_(mask.to(p.dtype) * 0.01)
    if rank == 0:
        stats.append(eng.send_weights(src.hf_named_tensors()))
    else:
        n = dst.load_hf_stream(eng.receive_weights())
        assert n == len(list(dst.parameters())), n
        for (k, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
            assert torch.equal(a, b), (step, k)
if rank == 0:
    torch.save(stats, os.environ["OUT"])
dist.barrier()
'''


def _run(tmp_path, backend, port):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    out = tmp_path / "stats.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), BACKEND=backend, OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return torch.load(out)


def test_bucketed_broadcast_delivers_every_tensor(tmp_path):
    stats = _run(tmp_path, "nccl", 29731)
    assert stats[0]["buckets"] > 1 and stats[0]["tensors"] > 10


def test_delta_sync_sends_only_changed_elements(tmp_path):
    stats = _run(tmp_path, "delta_sharded", 29732)
    assert stats[0]["dense"] == stats[0]["tensors"]                       # first sync is dense
    assert stats[1]["dense"] == 0 and stats[1]["changed_fraction"] < 0.03  # later ones are sparse
    assert stats[1]["bytes"] < 0.1 * stats[0]["bytes"]


def test_delta_compact_and_apply_roundtrip():
    g = torch.Generator().manual_seed(0)
    old = torch.randn(4096, generator=g).bfloat16()
    new = old.clone()
    idx = torch.randperm(4096, generator=g)[:37]
    new[idx] += 1.0
    snap, recv = old.clone(), old.clone()
    count, pos, val = delta_compact(new, snap)
    assert count == 37 and torch.equal(snap, new) and sorted(pos.tolist()) == sorted(idx.tolist())
    delta_apply(recv, pos, val)
    assert torch.equal(recv, new) and tensor_checksum(recv) == tensor_checksum(new)
    assert CheckpointEngineRegistry.get("naive") is not None


def test_fp8_blockwise_and_fp4_reference_formulas():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(200, 300, generator=g).bfloat16() * 3
    q, s = blockwise_cast_to_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
    assert torch.allclose(s[0, 0], x[:128, :128].float().abs().max() / 448)
    err = (dequant_blockwise_fp8(q, s).float() - x.float()).abs().max() / x.float().abs().max()
    assert err < 0.07
    w = torch.randn(8, 64, generator=g).bfloat16()
    y = fp4_fake_quant(w)
    grid = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6])
    ratio = (y.float().reshape(-1, 16).abs() / y.float().reshape(-1, 16).abs().amax(-1, keepdim=True).clamp_min(1e-9))
    assert y.shape == w.shape and (y.float() - w.float()).abs().max() < 0.6 and len(torch.unique(y.float().reshape(-1, 16)[0].abs())) <= 8
    w2 = w.clone().float().requires_grad_(True)
    fp4_fake_quant_ste(w2).sum().backward()
    assert torch.equal(w2.grad, torch.ones_like(w2))
    lin = QATLinear(torch.nn.Parameter(torch.randn(16, 32, generator=g)), mode="w4a4")
    out = lin(torch.randn(4, 32, generator=g))
    out.sum().backward()
    assert out.shape == (4, 16) and lin.weight.grad is not None and float(lin.weight_amax) > 0
