"""Checkpoint interchange with the reference's payload: per-rank ``{HF name: DTensor dim-0 shard}`` model files."""

import os
import subprocess
import sys

import pytest
import torch

from verl_b200.model_merger.__main__ import main as merger_main
from verl_b200.models.config import PRESETS
from verl_b200.models.hf_io import iter_safetensors
from verl_b200.utils.checkpoint.dtensor_interchange import is_named_tensor_payload, merge_sharded_model_files, saved_world_size
from verl_b200.workers.engine.fsdp.engine import FSDPEngine

# What the reference's FSDP2 engine does at save time, without the reference: shard every HF tensor on dim 0 over an ("fsdp",) mesh
# (optionally ("ddp", "fsdp")) with torch's own DTensor machinery and torch.save the per-rank dict; one buffer stays a plain tensor.
FOREIGN_WRITER = r'''
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.tensor import Replicate, Shard, distribute_tensor
from verl_b200.models.config import PRESETS
from verl_b200.models.transformer import DecoderLM
dist.init_process_group("gloo")
r, W = dist.get_rank(), dist.get_world_size()
hsdp = os.environ.get("HSDP") == "1"
mesh = init_device_mesh("cpu", (2, W // 2), mesh_dim_names=("ddp", "fsdp")) if hsdp else init_device_mesh("cpu", (W,), mesh_dim_names=("fsdp",))
pl = [Replicate(), Shard(0)] if hsdp else [Shard(0)]
model = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=11)
sd = {k: distribute_tensor(v.detach().clone(), mesh, pl) for k, v in model.hf_named_tensors()}
sd["model.rotary_emb.inv_freq"] = torch.arange(8.0)
os.makedirs(os.environ["OUT"], exist_ok=True)
torch.save(sd, os.path.join(os.environ["OUT"], f"model_world_size_{W}_rank_{r}.pt"))
if r == 0:
    json.dump({"FSDP_version": 2, "world_size": W}, open(os.path.join(os.environ["OUT"], "fsdp_config.json"), "w"))
dist.barrier()
'''

OWN_WRITER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.fsdp.engine import FSDPEngine
dist.init_process_group("gloo")
eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 4}, {"lr": 1e-3}, {"save_contents": ["model", "optimizer", "extra"], "model_format": "dtensor"})
eng.initialize()
eng.save_checkpoint(os.environ["OUT"], global_step=1)
if os.environ.get("RELOAD"):
    before = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    eng.store.flat.add_(1.0)
    eng.load_checkpoint(os.environ["OUT"])            # same world size: weights come back through the named-tensor path
    for n, p in eng.model.named_parameters():
        assert torch.equal(p, before[n]), n
    assert eng.step_count == 0 and float(eng.exp_avg.abs().sum()) == 0.0 and torch.equal(eng.master, eng.store.flat[eng.store.shard_slice].float())
dist.barrier()
'''


def _run(tmp_path, script_text, world, port, **env):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / f"w{port}.py"
    script.write_text(script_text)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(script)], env=dict(os.environ, REPO=repo, OMP_NUM_THREADS="1", **env), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("world,hsdp", [(3, False), (4, True)])
def test_a_checkpoint_in_the_foreign_payload_loads_into_the_engine_and_merges(tmp_path, world, hsdp):
    ck = tmp_path / "foreign"
    _run(tmp_path, FOREIGN_WRITER, world, 29871 + world, OUT=str(ck), HSDP="1" if hsdp else "0")
    assert saved_world_size(str(ck)) == world
    first = torch.load(ck / f"model_world_size_{world}_rank_0.pt", weights_only=False)
    assert is_named_tensor_payload(first) and not is_named_tensor_payload({"format": "flat_v1", "flat_shard": torch.zeros(1)})
    from verl_b200.models.transformer import DecoderLM

    want = dict(DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=11).hf_named_tensors())
    merged = merge_sharded_model_files(str(ck))
    assert set(merged) == set(want) | {"model.rotary_emb.inv_freq"}
    for k, v in want.items():
        assert torch.equal(merged[k], v), k               # uneven dim-0 shards (vocab 2048 / 3 ranks, norms of 64 rows) included
    # a single-process engine with other weights takes them over; the optimizer restarts from the loaded weights
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 4}, {"lr": 1e-3}, {"load_contents": ["model", "optimizer", "extra"]})
    eng.initialize()
    merged.pop("model.rotary_emb.inv_freq")
    os.remove(ck / f"model_world_size_{world}_rank_0.pt")
    first.pop("model.rotary_emb.inv_freq")
    torch.save(first, ck / f"model_world_size_{world}_rank_0.pt")     # (buffers are not parameters of this model: strict loading would refuse them)
    for r in range(1, world):
        sd = torch.load(ck / f"model_world_size_{world}_rank_{r}.pt", weights_only=False)
        sd.pop("model.rotary_emb.inv_freq")
        torch.save(sd, ck / f"model_world_size_{world}_rank_{r}.pt")
    eng.load_checkpoint(str(ck))
    got = dict(eng.model.hf_named_tensors())
    for k, v in want.items():
        assert torch.equal(got[k].float(), v), k
    assert torch.equal(eng.master, eng.store.flat[eng.store.shard_slice].float()) and eng.step_count == 0
    # the merger turns the same directory into HF safetensors
    PRESETS["tiny-qwen2"].save_pretrained(str(ck / "huggingface"))
    merger_main(["merge", "--backend", "fsdp", "--local_dir", str(ck), "--target_dir", str(tmp_path / "hf")])
    hf = dict(iter_safetensors(str(tmp_path / "hf")))
    for k, v in want.items():
        assert torch.equal(hf[k].float(), v.to(torch.bfloat16).float()), k


def test_the_engine_writes_the_foreign_payload_on_request(tmp_path):
    from torch.distributed.tensor import DTensor, Shard

    ck = tmp_path / "own"
    _run(tmp_path, OWN_WRITER, 2, 29879, OUT=str(ck), RELOAD="1")
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 4}, None, {})
    eng.initialize()
    want = dict(eng.model.hf_named_tensors())
    parts = [torch.load(ck / f"model_world_size_2_rank_{r}.pt", weights_only=False) for r in range(2)]
    assert set(parts[0]) == set(want)
    for k, v in want.items():
        a, b = parts[0][k], parts[1][k]
        # what the reference's merger does with the file: concatenate the local tensors along the recorded shard dimension
        assert isinstance(a, DTensor) and a.placements == (Shard(0),) and tuple(a.shape) == tuple(v.shape) and a.device_mesh.mesh_dim_names == ("fsdp",)
        assert torch.equal(torch.cat([a._local_tensor, b._local_tensor], dim=0), v.detach().cpu()), k
    import json

    assert json.load(open(ck / "fsdp_config.json"))["format"] == "dtensor"
    # one process loads the two-rank checkpoint (another world size): only this payload allows that
    eng2 = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 9}, {"lr": 1e-3}, {"load_contents": ["model"]})
    eng2.initialize()
    eng2.load_checkpoint(str(ck))
    for (n, a), (_, b) in zip(eng2.model.named_parameters(), eng.model.named_parameters()):
        assert torch.equal(a, b), n
