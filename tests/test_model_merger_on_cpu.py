import os
import subprocess
import sys

import torch

from verl_b200.model_merger.__main__ import main as merger_main
from verl_b200.models.config import PRESETS
from verl_b200.models.hf_io import iter_safetensors
from verl_b200.workers.engine.fsdp.engine import FSDPEngine

SAVE = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from verl_b200.models.config import PRESETS
from verl_b200.workers.engine.fsdp.engine import FSDPEngine
dist.init_process_group("gloo")
eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 4}, {"lr": 1e-3}, {"save_contents": ["model", "hf_model"]})
eng.initialize()
eng.save_checkpoint(os.environ["OUT"], global_step=1)
'''


def test_merge_two_rank_checkpoint_and_compare(tmp_path):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "save.py"
    script.write_text(SAVE)
    ck = tmp_path / "actor"
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29691", str(script)], env=dict(os.environ, REPO=repo, OUT=str(ck)), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert (ck / "model_world_size_2_rank_1.pt").exists()
    out = tmp_path / "merged"
    merger_main(["merge", "--backend", "fsdp", "--local_dir", str(ck), "--target_dir", str(out)])
    merged = dict(iter_safetensors(str(out)))
    eng = FSDPEngine(PRESETS["tiny-qwen2"], {"seed": 4}, None, {})
    eng.initialize()
    for name, t in eng.model.hf_named_tensors():
        assert torch.equal(merged[name].float(), t.to(torch.bfloat16).float()), name
    assert (out / "config.json").exists()
    # `test` compares against the HF export the engine wrote itself
    merger_main(["test", "--backend", "fsdp", "--local_dir", str(ck), "--test_hf_dir", str(ck / "huggingface")])
