"""Create a small randomly initialised HF-format checkpoint from a config (how the tests and smoke runs obtain tiny
models without network access): ``python -m verl_b200.scripts.init_random_model --preset qwen2.5-0.5b --num-layers 2
--out /tmp/tiny`` or ``--hf-config path/to/config.json`` (reference: ``scripts/init_random_model.py``)."""

from __future__ import annotations

import argparse
import json
import os

import torch

from verl_b200.models.config import PRESETS, ModelConfig
from verl_b200.models.hf_io import save_hf_checkpoint
from verl_b200.models.transformer import DecoderLM


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default=None)
    ap.add_argument("--hf-config", default=None)
    ap.add_argument("--override", default="{}", help="JSON dict of ModelConfig fields")
    ap.add_argument("--num-layers", type=int, default=None)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    cfg = PRESETS[a.preset] if a.preset else ModelConfig.from_pretrained(os.path.dirname(a.hf_config) if a.hf_config.endswith(".json") else a.hf_config)
    ov = json.loads(a.override)
    if a.num_layers is not None:
        ov["num_hidden_layers"] = a.num_layers
    cfg = cfg.replace(**ov) if ov else cfg
    model = DecoderLM(cfg, dtype=getattr(torch, a.dtype), seed=a.seed)
    save_hf_checkpoint(model, a.out)
    print(f"wrote {sum(p.numel() for p in model.parameters()) / 1e6:.1f}M-parameter {cfg.model_type} checkpoint to {a.out}")


if __name__ == "__main__":
    main()
