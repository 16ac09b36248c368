"""Cut a Hugging Face checkpoint into the sharded ``model/dist_ckpt`` files of the tensor/pipeline/data-parallel engine, so
that a large model starts from per-rank files instead of every rank reading (and slicing) the full weights.

    python -m verl_b200.scripts.converter_hf_to_mcore --hf_model_path <hf dir> --output_path <ckpt dir> \
        --tensor_model_parallel_size 2 --pipeline_model_parallel_size 2 --data_parallel_size 1

The output directory loads with ``MegatronCheckpointManager.load_checkpoint`` (model part only) and merges back with
``python -m verl_b200.model_merger merge --backend megatron``. Works on CPU; one (tp, pp) piece is alive at a time.

Reference: ``scripts/converter_hf_to_mcore.py`` (HF → Megatron-Core distributed checkpoint).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os

import torch

from verl_b200.models.config import ModelConfig
from verl_b200.models.hf_io import iter_safetensors
from verl_b200.models.parallel_model import local_model_config, local_to_global_name, shard_param, stage_layer_range
from verl_b200.models.transformer import DecoderLM, hf_to_native_state_dict
from verl_b200.utils.checkpoint.megatron_checkpoint_manager import shard_file
from verl_b200.workers.engine.fsdp.engine import FlatParamStore

__all__ = ["convert", "main"]


def convert(hf_model_path: str, output_path: str, tp: int = 1, pp: int = 1, dp: int = 1, dtype: torch.dtype = torch.bfloat16) -> dict:
    cfg = ModelConfig.from_pretrained(hf_model_path)
    native = hf_to_native_state_dict(cfg, dict(iter_safetensors(hf_model_path)))
    local_cfg = local_model_config(cfg, tp)
    os.makedirs(os.path.join(output_path, "model", "dist_ckpt"), exist_ok=True)
    written = 0
    for p in range(pp):
        layers = stage_layer_range(cfg.num_hidden_layers, pp, p)
        for t in range(tp):
            model = DecoderLM(local_cfg, dtype=dtype, device=torch.device("cpu"), init=False, layer_range=layers, pre_process=p == 0,
                              post_process=p == pp - 1) if tp * pp > 1 else DecoderLM(cfg, dtype=dtype, device=torch.device("cpu"), init=False)
            with torch.no_grad():
                for name, prm in model.named_parameters():
                    g = local_to_global_name(name, model.layer_offset)
                    if g not in native:
                        raise KeyError(f"{g} is not in the Hugging Face checkpoint")
                    src = native[g].to(dtype)
                    prm.copy_(shard_param(g, src, cfg, t, tp) if tp * pp > 1 else src)
            for d in range(dp):
                s = FlatParamStore(model, dp, d) if d == 0 else s_with_rank(s, d)
                torch.save({"format": "flat_mp_v1", "names": s.names, "shapes": [tuple(q.shape) for q in s.params], "offsets": s.offsets,
                            "total": s.total, "shard_size": s.shard_size, "dtype": str(s.flat.dtype), "tp_rank": t, "pp_rank": p, "dp_rank": d,
                            "layer_offset": model.layer_offset, "flat_shard": s.flat[s.shard_slice].detach().clone()},
                           shard_file(output_path, "model", t, p, d))
                written += 1
            del model
    hf_dir = os.path.join(output_path, "model", "huggingface")
    cfg.save_pretrained(hf_dir)
    for fn in os.listdir(hf_model_path):
        if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json", "generation_config.json"):
            import shutil

            shutil.copy(os.path.join(hf_model_path, fn), os.path.join(hf_dir, fn))
    meta = {"format": "flat_mp_v1", "tensor_model_parallel_size": tp, "pipeline_model_parallel_size": pp, "data_parallel_size": dp,
            "sequence_parallel": False,
            "stage_layers": [[r.start, r.stop] for r in (stage_layer_range(cfg.num_hidden_layers, pp, q) for q in range(pp))],
            "model_config": dataclasses.asdict(cfg)}
    with open(os.path.join(output_path, "transformer_config.json"), "w") as f:
        json.dump(meta, f, indent=2, default=str)
    with open(os.path.join(output_path, "ckpt_contents.json"), "w") as f:
        json.dump({"contents": ["model"], "global_step": 0}, f, indent=2)
    return {"files": written, **{k: meta[k] for k in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "data_parallel_size")}}


def s_with_rank(store: FlatParamStore, rank: int) -> FlatParamStore:
    """The same flat buffer seen from another data-parallel rank (only ``shard_slice`` depends on the rank)."""
    store.rank = rank
    return store


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--hf_model_path", required=True)
    ap.add_argument("--output_path", required=True)
    ap.add_argument("--tensor_model_parallel_size", type=int, default=1)
    ap.add_argument("--pipeline_model_parallel_size", type=int, default=1)
    ap.add_argument("--data_parallel_size", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    a = ap.parse_args(argv)
    out = convert(a.hf_model_path, a.output_path, a.tensor_model_parallel_size, a.pipeline_model_parallel_size, a.data_parallel_size,
                  getattr(torch, a.dtype))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
