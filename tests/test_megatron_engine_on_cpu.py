"""TP × PP × DP engine on gloo ranks: log-probs, gradients, gradient norm and exported weights equal the single-rank run."""

import os
import subprocess
import sys

import pytest
import torch

from tests.test_engine_on_cpu import loss_fn, make_batch
from verl_b200.models.config import PRESETS
from verl_b200.models.parallel_model import local_model_config, shard_param, stage_layer_range, unshard_param
from verl_b200.models.transformer import DecoderLM
from verl_b200.workers.engine.fsdp.engine import FSDPEngine

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from tests.test_engine_on_cpu import make_batch, loss_fn
from verl_b200.models.config import PRESETS
from verl_b200.models.parallel_model import local_to_global_name, tp_rule, unshard_param
from verl_b200.workers.engine.megatron.engine import MegatronEngine
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cfg = PRESETS["tiny-qwen2"].replace(num_hidden_layers=int(os.environ.get("LAYERS", "3")), tie_word_embeddings=os.environ["TIED"] == "1")
eng = MegatronEngine(cfg, {"seed": 1, "tensor_model_parallel_size": int(os.environ["TP"]), "pipeline_model_parallel_size": int(os.environ["PP"]),
                           "virtual_pipeline_model_parallel_size": int(os.environ.get("VPP", "1")),
                           "sequence_parallel": os.environ.get("SP", "0") == "1", "context_parallel_size": int(os.environ.get("CP", "1")),
                           "context_parallel_zigzag": os.environ.get("ZIGZAG", "0") == "1"},
                     {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
eng.initialize()
exported = {k: v.clone() for k, v in eng.get_per_tensor_param()[0]}
data = make_batch().chunk(eng.get_data_parallel_size())[eng.get_data_parallel_rank()]
data.meta_info["micro_batch_size_per_gpu"] = int(os.environ.get("MBS", "2"))
lp = eng.infer_batch(data)["model_output"]["log_probs"]
eng.optimizer_zero_grad()
out = eng.forward_backward_batch(data, loss_fn)
ent = out["model_output"]["entropy"]
grads = {}
for n, p in eng.model.named_parameters():
    g = eng._gname(n)
    mg = p.main_grad.clone()
    if eng.fsdp_size > 1:
        dist.all_reduce(mg, group=eng.fsdp_group); mg /= eng.fsdp_size
    if eng.tp_size > 1 and tp_rule(g, cfg) is not None:
        parts = [torch.empty_like(mg) for _ in range(eng.tp_size)]
        dist.all_gather(parts, mg, group=eng.tp_group)
        mg = unshard_param(g, parts, cfg)
    grads[g] = mg
gn = eng.optimizer_step()
after = None
if os.environ.get("CKPT"):
    # Megatron-layout checkpoint: save, take another step, reload -> parameters and optimizer state are back
    eng.save_checkpoint(os.environ["CKPT"], global_step=1)
    after = {k: v.clone() for k, v in eng.get_per_tensor_param()[0]}
    flat0, m0, step0 = eng.store.flat.clone(), eng.exp_avg.clone(), eng.step_count
    eng.optimizer_zero_grad(); eng.forward_backward_batch(data, loss_fn); eng.optimizer_step()
    assert not torch.equal(eng.store.flat, flat0)
    eng.load_checkpoint(os.environ["CKPT"])
    assert torch.equal(eng.store.flat, flat0) and torch.equal(eng.exp_avg, m0) and eng.step_count == step0
torch.save({"grads": grads, "after": after if rank == 0 else None, "gn": gn, "lp": lp, "ent": ent, "dp_rank": eng.dp_rank, "exported": exported if rank == 0 else None,
            "src": eng.is_mp_src_rank_with_outputs()}, os.environ["OUT"] + f".{rank}")
dist.barrier()
'''


def test_shard_unshard_roundtrip():
    cfg = PRESETS["tiny-qwen2"]
    full = DecoderLM(cfg, dtype=torch.float32, seed=3)
    for name, p in full.named_parameters():
        parts = [shard_param(name, p, cfg, r, 2) for r in range(2)]
        assert torch.equal(unshard_param(name, parts, cfg), p), name
    lc = local_model_config(cfg, 2)
    local = DecoderLM(lc, dtype=torch.float32, init=False)
    for name, p in local.named_parameters():
        assert tuple(shard_param(name, dict(full.named_parameters())[name], cfg, 1, 2).shape) == tuple(p.shape), name
    assert [list(stage_layer_range(7, 3, s)) for s in range(3)] == [[0, 1, 2], [3, 4], [5, 6]]


@pytest.mark.parametrize("world,tp,pp,tied,sp,cp,zigzag,vpp,layers,mbs", [
    (4, 2, 2, False, False, 1, False, 1, 3, 2), (4, 1, 2, True, False, 1, False, 1, 3, 2), (3, 1, 3, True, False, 1, False, 1, 3, 2),
    (2, 2, 1, True, False, 1, False, 1, 3, 2), (2, 2, 1, False, True, 1, False, 1, 3, 2), (4, 2, 2, True, True, 1, False, 1, 3, 2),
    # context parallelism: with TP, with PP (zig-zag), with sequence-parallel TP, and with DP on top
    (4, 2, 1, True, False, 2, False, 1, 3, 2), (4, 1, 2, False, False, 2, True, 1, 3, 2), (4, 2, 1, False, True, 2, False, 1, 3, 2),
    (4, 1, 1, True, False, 2, True, 1, 3, 2),
    # virtual pipeline stages (interleaved 1F1B): 2 ranks x 2 chunks with tied embeddings; with TP and an uneven layer split; three ranks
    # with a micro-batch count that is not a multiple of the pipeline depth
    (2, 1, 2, True, False, 1, False, 2, 4, 2), (4, 2, 2, False, False, 1, False, 2, 5, 3), (3, 1, 3, True, False, 1, False, 2, 6, 3),
    # virtual stages together with zig-zag context parallelism
    (4, 1, 2, False, False, 2, True, 2, 4, 2)])
def test_parallel_ranks_match_single_rank(tmp_path, world, tp, pp, tied, sp, cp, zigzag, vpp, layers, mbs):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    out = tmp_path / "out.pt"
    env = dict(os.environ, REPO=repo, OUT=str(out), OMP_NUM_THREADS="1", TP=str(tp), PP=str(pp), TIED="1" if tied else "0", SP="1" if sp else "0", CP=str(cp),
               ZIGZAG="1" if zigzag else "0", VPP=str(vpp), LAYERS=str(layers), MBS=str(mbs))
    ckpt = tmp_path / "ckpt"
    if (world, tp, pp) in ((4, 2, 2), (4, 1, 2)) and not sp:
        env["CKPT"] = str(ckpt)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29660 + world + tp + (10 if sp else 0) + 20 * (cp - 1) + (5 if zigzag else 0) + 40 * (vpp - 1)), str(script)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    cfg = PRESETS["tiny-qwen2"].replace(num_hidden_layers=layers, tie_word_embeddings=tied)
    eng = FSDPEngine(cfg, {"seed": 1}, {"lr": 1e-3, "weight_decay": 0.01, "clip_grad": 1.0}, {})
    eng.initialize()
    data = make_batch()
    data.meta_info["micro_batch_size_per_gpu"] = mbs
    lp = eng.infer_batch(data)["model_output"]["log_probs"]
    eng.optimizer_zero_grad()
    ent = eng.forward_backward_batch(data, loss_fn)["model_output"]["entropy"]
    ref_grads = {n: p.main_grad.clone() for n, p in eng.model.named_parameters()}
    gn = eng.optimizer_step()
    res = [torch.load(str(out) + f".{r}") for r in range(world)]
    dp = world // (tp * pp * cp)
    per = len(data) // dp
    seen = set()
    for r in res:
        sl = slice(r["dp_rank"] * per, (r["dp_rank"] + 1) * per)
        assert torch.allclose(r["lp"], lp[sl], atol=2e-5), (r["lp"] - lp[sl]).abs().max()
        assert torch.allclose(r["ent"], ent[sl], atol=2e-5)
        assert abs(r["gn"] - gn) < 1e-4 * max(1.0, gn), (r["gn"], gn)
        for n, g in r["grads"].items():
            assert torch.allclose(g, ref_grads[n], atol=2e-6, rtol=1e-4), (n, (g - ref_grads[n]).abs().max())
            seen.add(n)
    assert seen == set(ref_grads)
    assert sum(r["src"] for r in res) == dp
    fresh = DecoderLM(cfg, dtype=torch.float32, seed=1)
    want = dict(fresh.hf_named_tensors())
    assert set(res[0]["exported"]) == set(want)
    for k, v in want.items():
        assert torch.equal(res[0]["exported"][k], v), k
    if "CKPT" in env:
        # the merger rebuilds parallelism-independent HF weights from the (tp, pp, dp) shards
        for f in ("transformer_config.json", "ckpt_contents.json", "model/huggingface/config.json", "model/dist_ckpt/shard_tp0_pp1_dp0.pt",
                  "optimizer/dist_ckpt/shard_tp0_pp0_dp0.pt", "extra/dist_ckpt/shard_tp0_pp0_dp0.pt"):
            assert (ckpt / f).exists(), f
        from safetensors.torch import load_file

        from verl_b200.model_merger.__main__ import main as merger_main

        merger_main(["merge", "--backend", "megatron", "--local_dir", str(ckpt), "--target_dir", str(tmp_path / "hf")])
        merged = {}
        for fn in os.listdir(tmp_path / "hf"):
            if fn.endswith(".safetensors"):
                merged.update(load_file(str(tmp_path / "hf" / fn)))
        after = res[0]["after"]
        assert set(merged) == set(after)
        for k, v in after.items():
            assert torch.equal(merged[k].float(), v.to(torch.bfloat16).float()), k


def test_grpo_fit_with_tensor_and_pipeline_parallel_actor(tmp_path):
    """main_ppo under torchrun with strategy=megatron: tp=2 for actor and ref (dp=1 ⇒ both ranks see the whole batch),
    rollout replicas refreshed from the per-tensor export."""
    import json

    from tests.test_trainer_e2e_on_cpu import OV

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    logf = tmp_path / "log.jsonl"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29677",
           "-m", "verl_b200.trainer.main_ppo"] + [o for o in OV if not o.startswith("trainer.logger")] + \
          ["trainer.logger=[file]", "trainer.total_training_steps=2", f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.resume_mode=disable",
           "actor_rollout_ref.actor.strategy=megatron", "actor_rollout_ref.ref.strategy=megatron",
           "actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2", "actor_rollout_ref.ref.megatron.tensor_model_parallel_size=2"]
    env = dict(os.environ, VERL_FILE_LOGGER_PATH=str(logf), OMP_NUM_THREADS="2", PYTHONPATH=repo)
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=repo)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rows = [json.loads(x) for x in logf.read_text().splitlines()]
    assert len(rows) == 2 and rows[-1]["data"]["perf/total_num_tokens"] > 0 and abs(rows[0]["data"]["actor/ppo_kl"]) < 1e-4
    assert abs(rows[0]["data"]["rollout_corr/kl"] if "rollout_corr/kl" in rows[0]["data"] else 0.0) < 1e-3


def test_hf_to_sharded_converter_round_trips_through_the_merger(tmp_path):
    """HF checkpoint → (tp=2, pp=2, dp=2) shard files → merger → the same HF tensors."""
    from verl_b200.models.config import PRESETS
    from verl_b200.models.hf_io import iter_safetensors, save_hf_checkpoint
    from verl_b200.models.transformer import DecoderLM
    from verl_b200.model_merger.__main__ import main as merger_main
    from verl_b200.scripts.converter_hf_to_mcore import main as convert_main

    cfg = PRESETS["tiny-qwen2"]
    model = DecoderLM(cfg, dtype=torch.float32, seed=3)
    src = tmp_path / "hf_src"
    save_hf_checkpoint(model, str(src), dtype=torch.float32)
    out = tmp_path / "sharded"
    convert_main(["--hf_model_path", str(src), "--output_path", str(out), "--tensor_model_parallel_size", "2",
                  "--pipeline_model_parallel_size", "2", "--data_parallel_size", "2", "--dtype", "float32"])
    assert len(os.listdir(out / "model" / "dist_ckpt")) == 8
    merger_main(["merge", "--backend", "megatron", "--local_dir", str(out), "--target_dir", str(tmp_path / "hf_back")])
    want, got = dict(iter_safetensors(str(src))), dict(iter_safetensors(str(tmp_path / "hf_back")))
    assert want.keys() == got.keys()
    for k in want:
        assert torch.allclose(got[k].float(), want[k].float(), atol=1e-2, rtol=1e-2), k
