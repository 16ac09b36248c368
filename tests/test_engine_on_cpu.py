"""fsdp engine on CPU: sharded optimizer equals a plain torch AdamW run; two gloo ranks equal one rank."""

import os
import subprocess
import sys
import tempfile

import pytest
import torch

from verl_b200.models.config import PRESETS
from verl_b200.models.transformer import DecoderLM, PackedBatch
from verl_b200.protocol import DataProto
from verl_b200.workers.engine.fsdp.engine import FSDPEngine
from verl_b200.workers.utils.losses import ppo_loss

ACTOR_CFG = {"clip_ratio": 0.2, "use_kl_loss": True, "kl_loss_coef": 1e-3, "entropy_coeff": 0.0, "loss_agg_mode": "token-mean"}


def make_batch(bs=8, P=12, R=10, vocab=2048, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(10, vocab, (bs, P + R), generator=g)
    att = torch.ones(bs, P + R, dtype=torch.int64)
    for i in range(bs):
        att[i, : int(torch.randint(0, 5, (1,), generator=g))] = 0
        k = int(torch.randint(0, 4, (1,), generator=g))
        if k:
            att[i, -k:] = 0
    pos = torch.clip(torch.cumsum(att, -1) - 1, min=0)
    return DataProto.from_dict(tensors={
        "input_ids": ids, "attention_mask": att, "position_ids": pos, "responses": ids[:, -R:], "response_mask": att[:, -R:],
        "old_log_probs": -7.6 + 0.1 * torch.randn(bs, R, generator=g), "ref_log_prob": -7.6 + 0.1 * torch.randn(bs, R, generator=g),
        "advantages": torch.randn(bs, R, generator=g)}, meta_info={"micro_batch_size_per_gpu": 3, "temperature": 1.0, "calculate_entropy": True})


def loss_fn(model_output, data, dp_group=None):
    return ppo_loss(ACTOR_CFG, model_output, data)


def test_infer_matches_direct_forward():
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, None, {})
    eng.initialize()
    data = make_batch()
    out = eng.infer_batch(data)["model_output"]
    b = data.batch
    for i in range(len(data)):
        m = b["attention_mask"][i].bool()
        ids = b["input_ids"][i][m]
        pb = PackedBatch(ids, torch.arange(len(ids), dtype=torch.int32), torch.tensor([0, len(ids)], dtype=torch.int32))
        with torch.no_grad():
            logits = eng.model(pb, return_logits=True)["logits"]
        lp = torch.log_softmax(logits.float(), -1)
        R = b["responses"].shape[1]
        p_len = int(b["attention_mask"][i, :-R].sum())
        r_len = int(b["attention_mask"][i, -R:].sum())
        for t in range(r_len):
            want = lp[p_len - 1 + t, ids[p_len + t]]
            assert abs(out["log_probs"][i, t] - want) < 1e-4
        assert (out["log_probs"][i, r_len:] == 0).all()


def _ref_grads(data, seed=1):
    """Gradients of the same loss through plain autograd on a packed forward of the whole batch."""
    from verl_b200.workers.utils.padding import response_gather_index

    ref = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=seed)
    b = data.batch
    att = b["attention_mask"].bool()
    ids, pos, lens = b["input_ids"][att], b["position_ids"][att], att.sum(-1)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    logits = ref(PackedBatch(ids, pos.to(torch.int32), cu), return_logits=True)["logits"]
    lp_all = torch.log_softmax(logits.float(), -1).gather(-1, torch.roll(ids, -1)[:, None]).squeeze(-1)
    idx, valid = response_gather_index(b["attention_mask"], b["responses"].shape[1])
    lp = torch.where(valid, lp_all[idx.reshape(-1)].reshape(idx.shape), torch.zeros(()))
    loss, _ = ppo_loss(ACTOR_CFG, {"log_probs": lp}, dict(b.items()))
    loss.backward()
    return ref


def test_gradients_match_autograd_and_are_micro_batch_invariant():
    data = make_batch()
    ref = _ref_grads(data)
    for mbs in (8, 3):
        eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3}, {})
        eng.initialize()
        data.meta_info["micro_batch_size_per_gpu"] = mbs
        eng.optimizer_zero_grad()
        eng.forward_backward_batch(data, loss_fn)
        for (n, p), (_, q) in zip(eng.model.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p.main_grad, q.grad, atol=1e-6, rtol=1e-4), (mbs, n, (p.main_grad - q.grad).abs().max())


def test_dynamic_bsz_gives_same_gradients():
    data = make_batch()
    ref = _ref_grads(data)
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3}, {})
    eng.initialize()
    data.meta_info.update({"use_dynamic_bsz": True, "max_token_len_per_gpu": 50})
    eng.optimizer_zero_grad()
    out = eng.forward_backward_batch(data, loss_fn)
    assert len(out["loss"]) >= 3
    for (n, p), (_, q) in zip(eng.model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.main_grad, q.grad, atol=1e-6, rtol=1e-4), n


def test_optimizer_step_matches_torch_adamw():
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
    eng.initialize()
    ref = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=1)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.01)
    g = torch.Generator().manual_seed(5)
    for step in range(3):
        eng.optimizer_zero_grad()
        for p, q in zip(eng.model.parameters(), ref.parameters()):
            gr = torch.randn(q.shape, generator=g) * 0.5
            p.main_grad.copy_(gr)
            q.grad = gr.clone()
        gn_ref = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        gn = eng.optimizer_step()
        assert abs(gn - float(gn_ref)) < 1e-3
        for p, q in zip(eng.model.parameters(), ref.parameters()):
            assert torch.allclose(p, q, atol=1e-6)


def test_nonfinite_grad_skips_step():
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3}, {})
    eng.initialize()
    before = eng.store.flat.clone()
    eng.optimizer_zero_grad()
    eng.store.grad.fill_(float("nan"))
    gn = eng.optimizer_step()
    assert gn != gn and torch.equal(eng.store.flat, before) and eng.step_count == 0


def test_checkpoint_roundtrip_and_hf_export(tmp_path):
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3}, {"save_contents": ["model", "optimizer", "extra", "hf_model"]})
    eng.initialize()
    eng.train_batch(make_batch(), loss_fn)
    eng.lr_scheduler_step()
    eng.save_checkpoint(str(tmp_path / "actor"), global_step=1)
    assert (tmp_path / "actor" / "model_world_size_1_rank_0.pt").exists() and (tmp_path / "actor" / "fsdp_config.json").exists()
    assert (tmp_path / "actor" / "huggingface" / "config.json").exists() and (tmp_path / "actor" / "huggingface" / "model.safetensors").exists()
    eng2 = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 9}, {"lr": 1e-3}, {})
    eng2.initialize()
    eng2.load_checkpoint(str(tmp_path / "actor"))
    assert torch.equal(eng2.store.flat, eng.store.flat) and torch.equal(eng2.exp_avg, eng.exp_avg) and eng2.step_count == 1 and eng2.sched_step == 1
    from verl_b200.models.hf_io import iter_safetensors

    sd = dict(iter_safetensors(str(tmp_path / "actor" / "huggingface")))
    assert torch.allclose(sd["model.embed_tokens.weight"].float(), eng.model.embed_tokens.float(), atol=1e-2)


WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from tests.test_engine_on_cpu import make_batch, loss_fn
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.fsdp.engine import FSDPEngine
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
eng.initialize()
data = make_batch().chunk(world)[rank]
data.meta_info["micro_batch_size_per_gpu"] = 2
out = eng.train_batch(data, loss_fn)
if rank == 0:
    torch.save({"flat": eng.store.flat, "gn": out["metrics"]["grad_norm"]}, os.environ["OUT"])
dist.barrier()
'''


def test_two_gloo_ranks_match_single_rank(tmp_path):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    out = tmp_path / "out.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29653", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    two = torch.load(out)
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 1}, {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
    eng.initialize()
    o = eng.train_batch(make_batch(), loss_fn)
    n = min(eng.store.flat.numel(), two["flat"].numel())
    assert abs(o["metrics"]["grad_norm"] - two["gn"]) < 1e-4
    # Adam's first step is sign-like for near-zero gradients, so compare within one learning-rate quantum
    assert (eng.store.flat[:n] - two["flat"][:n]).abs().max() <= 2.1e-3
    assert ((eng.store.flat[:n] - two["flat"][:n]).abs() > 1e-6).float().mean() < 0.02


def test_tiled_mlp_matches_the_dense_mlp_and_frees_activations():
    """`model.tiled_mlp.enabled`: outputs, input gradients and weight gradients (accumulated into main_grad over the tiles) equal
    the untiled run; only the MLP input is saved for backward."""
    from verl_b200.models.transformer import _tile_bounds

    assert _tile_bounds(10, 4) == [(0, 3), (3, 6), (6, 9), (9, 10)] and _tile_bounds(1100, 4) == [(0, 384), (384, 768), (768, 1100)]
    res = {}
    for tiled in (False, True):
        mc = {"preset": "tiny-qwen2", "tiled_mlp": {"enabled": tiled, "num_shards": 3}}
        eng = FSDPEngine(mc, {"seed": 1}, {"lr": 1e-3, "clip_grad": 1.0}, {})
        eng.initialize()
        assert eng.model.layers[0].mlp.tiled_shards == (3 if tiled else 0)
        data = make_batch()
        lp = eng.infer_batch(data)["model_output"]["log_probs"]
        eng.optimizer_zero_grad()
        eng.forward_backward_batch(data, loss_fn)
        res[tiled] = (lp, eng.store.grad.clone(), eng.optimizer_step())
    assert torch.allclose(res[True][0], res[False][0], atol=1e-6)
    assert torch.allclose(res[True][1], res[False][1], atol=1e-6, rtol=1e-4)
    assert abs(res[True][2] - res[False][2]) < 1e-5
