"""ZeRO-3 mode of the fsdp engine on gloo ranks: same log-probs, gradient norms, weights and merged checkpoint as one rank
holding everything.

Reference behaviour: FSDP FULL_SHARD (verl/workers/engine/fsdp/transformer_impl.py:389-498)."""

import os
import subprocess
import sys

import pytest
import torch

from tests.test_engine_on_cpu import loss_fn, make_batch
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.base import EngineRegistry
from verl_b200.workers.engine.fsdp.engine import FSDPEngine

OPT = {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from tests.test_engine_on_cpu import make_batch, loss_fn
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.base import EngineRegistry
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
eng = EngineRegistry.new("language_model", "fsdp", model_config=PRESETS["tiny-qwen2"], engine_config={"seed": 1, "reshard_after_forward": True},
                         optimizer_config={"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, checkpoint_config={"save_contents": ["model", "optimizer", "extra", "hf_model"]})
eng.initialize()
assert type(eng).__name__ == "Zero3Engine" and eng.get_data_parallel_size() == world
cfg = eng.cfg
qkv = dict(eng.model.named_parameters())["layers.0.self_attn.qkv_proj"]
assert qkv.shape[0] * world == cfg.q_size + 2 * cfg.kv_size, qkv.shape
data = make_batch().chunk(world)[rank]
data.meta_info["micro_batch_size_per_gpu"] = 3
lp = eng.infer_batch(data)["model_output"]["log_probs"]
gns = []
for _ in range(2):
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(data, loss_fn)
    gns.append(eng.optimizer_step())
tensors = {k: v.detach().clone() for k, v in eng.get_per_tensor_param()[0]}
eng.save_checkpoint(os.environ["OUT"] + ".ckpt", global_step=2)
# a reload restores weights and optimizer state of the shards
before = eng.store.flat.clone()
eng.store.flat.zero_()
eng.load_checkpoint(os.environ["OUT"] + ".ckpt")
assert torch.equal(eng.store.flat, before)
torch.save({"lp": lp, "gns": gns, "tensors": tensors}, os.environ["OUT"] + f".{rank}")
dist.barrier()
'''


@pytest.mark.parametrize("world", [2, 4])
def test_zero3_ranks_match_single_rank(tmp_path, world):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    out = tmp_path / "out.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29790 + world), str(script)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, OPT, {})
    eng.initialize()
    data = make_batch()
    data.meta_info["micro_batch_size_per_gpu"] = 3
    lp = eng.infer_batch(data)["model_output"]["log_probs"]
    gns = []
    for _ in range(2):
        eng.optimizer_zero_grad()
        eng.forward_backward_batch(data, loss_fn)
        gns.append(eng.optimizer_step())
    want = {k: v.detach().clone() for k, v in eng.get_per_tensor_param()[0]}
    per = len(data) // world
    for rk in range(world):
        res = torch.load(str(out) + f".{rk}")
        assert torch.allclose(res["lp"], lp[rk * per:(rk + 1) * per], atol=2e-5)
        for a, b in zip(res["gns"], gns):
            assert abs(a - b) < 1e-4 * max(1.0, b), (res["gns"], gns)
        assert res["tensors"].keys() == want.keys()
        for k in want:
            assert res["tensors"][k].shape == want[k].shape, k
            # AdamW normalises the step, so fp32 summation-order noise in a near-zero gradient moves a weight by up to ~lr
            d = (res["tensors"][k] - want[k]).abs()
            assert d.max() < 2.5e-3 and d.mean() < 2e-5, (k, float(d.max()), float(d.mean()))
    # per-rank files merge back into the full weights; the collective HF export wrote the same tensors
    from verl_b200.model_merger.base_model_merger import ModelMergerConfig
    from verl_b200.model_merger.fsdp_model_merger import FSDPModelMerger

    ckpt = str(out) + ".ckpt"
    merger = FSDPModelMerger(ModelMergerConfig(operation="merge", backend="fsdp", local_dir=ckpt, target_dir=str(tmp_path / "hf"),
                                               hf_model_config_path=os.path.join(ckpt, "huggingface")))
    sd = merger._merge()
    for k in want:
        assert torch.allclose(sd[k].float(), want[k].float(), atol=1e-2, rtol=1e-2), k
    from verl_b200.models.hf_io import iter_safetensors

    hf = dict(iter_safetensors(os.path.join(ckpt, "huggingface")))
    for k in want:
        assert torch.allclose(hf[k].float(), want[k].float(), atol=1e-2, rtol=1e-2), k


def test_zero3_single_rank_is_plain_engine():
    eng = EngineRegistry.new("language_model", "fsdp", model_config=PRESETS["tiny-qwen2"], engine_config={"seed": 1, "zero3": True},
                             optimizer_config=OPT, checkpoint_config={})
    eng.initialize()
    ref = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, OPT, {})
    ref.initialize()
    data = make_batch()
    for e in (eng, ref):
        e.optimizer_zero_grad()
        e.forward_backward_batch(data, loss_fn)
    a, b = eng.optimizer_step(), ref.optimizer_step()
    assert abs(a - b) < 1e-5 * max(1.0, b)
    got, want = dict(eng.get_per_tensor_param()[0]), dict(ref.get_per_tensor_param()[0])
    for k in want:
        assert torch.allclose(got[k], want[k], atol=1e-6), k


MOE_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from tests.test_engine_on_cpu import make_batch, loss_fn
from tests.test_zero3_on_cpu import moe_config
from verl_b200.workers.engine.base import EngineRegistry
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
if os.environ["DENSE"] == "2":      # the Megatron-style names of the same layout: strategy megatron, expert_model_parallel_size = world
    eng = EngineRegistry.new("language_model", "megatron", model_config=moe_config(), engine_config={"seed": 1, "expert_model_parallel_size": world,
                             "tensor_model_parallel_size": 1, "pipeline_model_parallel_size": 1}, optimizer_config={"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0},
                             checkpoint_config={})
    try:
        EngineRegistry.new("language_model", "megatron", model_config=moe_config(), engine_config={"expert_model_parallel_size": world, "tensor_model_parallel_size": 2})
        raise SystemExit("expert parallelism combined with tensor parallelism must be refused")
    except NotImplementedError:
        pass
else:
    eng = EngineRegistry.new("language_model", "fsdp", model_config=moe_config(), engine_config={"seed": 1, "expert_parallel_size": world,
                             "zero3": os.environ["DENSE"] == "1"}, optimizer_config={"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, checkpoint_config={})
eng.initialize()
assert type(eng).__name__ == "Zero3Engine"
gu = dict(eng.model.named_parameters())["layers.0.mlp.experts_gate_up"]
assert gu.shape[0] == 4 // world and eng.model.layers[0].mlp.ep_group is not None
data = make_batch(vocab=512).chunk(world)[rank]
data.meta_info["micro_batch_size_per_gpu"] = 3
lp = eng.infer_batch(data)["model_output"]["log_probs"]
gns = []
for _ in range(2):
    eng.optimizer_zero_grad()
    eng.forward_backward_batch(data, loss_fn)
    gns.append(eng.optimizer_step())
tensors = {k: v.detach().clone() for k, v in eng.get_per_tensor_param()[0]}
torch.save({"lp": lp, "gns": gns, "tensors": tensors}, os.environ["OUT"] + f".{rank}")
dist.barrier()
"""


def moe_config():
    from verl_b200.models.config import ModelConfig

    return ModelConfig(model_type="qwen3_moe", vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, attention_bias=False, qk_norm=True, num_experts=4, num_experts_per_tok=2,
                       moe_intermediate_size=32, rope_theta=1e4, max_position_embeddings=512, torch_dtype="float32")


@pytest.mark.parametrize("dense", [0, 1, 2])
def test_expert_parallel_ranks_match_single_rank(tmp_path, dense):
    """Experts spread over two ranks (tokens reach them by all-to-all), alone and together with row-sharded projections:
    log-probs, gradient norms and exported weights equal a single rank holding every expert."""
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(MOE_WORKER)
    out = tmp_path / "out.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1", DENSE=str(dense))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", str(29796 + dense), str(script)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    eng = FSDPEngine(moe_config(), {"seed": 1}, OPT, {})
    eng.initialize()
    data = make_batch(vocab=512)
    data.meta_info["micro_batch_size_per_gpu"] = 3
    lp = eng.infer_batch(data)["model_output"]["log_probs"]
    gns = []
    for _ in range(2):
        eng.optimizer_zero_grad()
        eng.forward_backward_batch(data, loss_fn)
        gns.append(eng.optimizer_step())
    want = {k: v.detach().clone() for k, v in eng.get_per_tensor_param()[0]}
    per = len(data) // 2
    for rk in range(2):
        res = torch.load(str(out) + f".{rk}")
        assert torch.allclose(res["lp"], lp[rk * per:(rk + 1) * per], atol=2e-5)
        for a, b in zip(res["gns"], gns):
            assert abs(a - b) < 1e-4 * max(1.0, b), (res["gns"], gns)
        assert res["tensors"].keys() == want.keys()
        for k in want:
            d = (res["tensors"][k] - want[k]).abs()
            assert res["tensors"][k].shape == want[k].shape and d.max() < 2.5e-3 and d.mean() < 2e-5, (k, float(d.max()), float(d.mean()))


VL_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.base import EngineRegistry
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
eng = EngineRegistry.new("language_model", "fsdp", model_config=PRESETS["tiny-qwen2-vl"], engine_config={"seed": 1, "zero3": True},
                         optimizer_config={"lr": 1e-3}, checkpoint_config={})
eng.initialize()
named = dict(eng.model.named_parameters())
assert named["language_model.layers.0.mlp.gate_up_proj"].shape[0] == 1024 // world and named["visual.blocks.0.attn.qkv.weight"].shape[0] == 96
tensors = {k: v.detach().clone() for k, v in eng.get_per_tensor_param()[0]}
torch.save(tensors, os.environ["OUT"] + f".{rank}")
dist.barrier()
"""


def test_zero3_shards_the_decoder_of_a_vision_language_model(tmp_path):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(VL_WORKER)
    out = tmp_path / "out.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29799", str(script)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    eng = FSDPEngine(PRESETS["tiny-qwen2-vl"], {"seed": 1}, OPT, {})
    eng.initialize()
    want = dict(eng.get_per_tensor_param()[0])
    got = torch.load(str(out) + ".1")
    assert got.keys() == want.keys() and "visual.merger.mlp.2.weight" in got
    for k in want:
        assert got[k].shape == want[k].shape and torch.equal(got[k], want[k]), k
