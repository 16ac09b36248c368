"""Fold a LoRA checkpoint into its base model and export both forms.

    python -m verl_b200.scripts.merge_lora --base_model /models/Qwen2.5-7B --local_dir ckpt/global_step_100/actor --target_dir out/merged

A LoRA run's sharded checkpoint holds the adapters only (they are the engine's whole parameter store). This tool rebuilds the
flat buffer from the per-rank shards, attaches the adapters to the base weights (a Hugging Face directory or a preset name) and
writes (a) ``target_dir/``: full HF safetensors with the update folded in, and (b) ``target_dir/lora_adapter/``: the adapters in
the PEFT layout (``adapter_model.safetensors`` + ``adapter_config.json``; the fused qkv / gate_up adapters are split per HF module:
the modules of a fused projection share ``lora_A`` and take their rows of ``lora_B``).

Reference: ``scripts/megatron_merge_lora.py`` (merged HF weights written next to the adapter checkpoint through a worker group) and
the ``lora_adapter`` export of ``verl/model_merger/fsdp_model_merger.py``.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

__all__ = ["merge_lora_checkpoint", "main"]


def _load_adapters(local_dir: str) -> tuple[dict, dict]:
    with open(os.path.join(local_dir, "fsdp_config.json")) as f:
        meta = json.load(f)
    if "lora" not in meta:
        raise ValueError(f"{local_dir} was not written by a LoRA run (no 'lora' entry in fsdp_config.json)")
    world = int(meta["world_size"])
    first = torch.load(os.path.join(local_dir, f"model_world_size_{world}_rank_0.pt"), map_location="cpu", weights_only=False)
    n = int(first["fsdp_size"])
    shards = [first] + [torch.load(os.path.join(local_dir, f"model_world_size_{world}_rank_{r}.pt"), map_location="cpu", weights_only=False)
                        for r in range(1, n)]
    shards.sort(key=lambda s: s["fsdp_rank"])
    flat = torch.cat([s["flat_shard"] for s in shards])
    out = {}
    for name, shape, off in zip(first["names"], first["shapes"], first["offsets"]):
        k = 1
        for d in shape:
            k *= d
        out[name] = flat[off: off + k].view(*shape)
    return out, meta["lora"]


def _peft_tensors(cfg, adapters: dict) -> dict:
    """Native adapter names (``layers.i.self_attn.lora_A_qkv_proj``) → PEFT names on the HF modules."""
    q, kv, inter = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim, cfg.intermediate_size
    split = {"qkv_proj": (("q_proj", 0, q), ("k_proj", q, q + kv), ("v_proj", q + kv, q + 2 * kv)), "o_proj": (("o_proj", 0, None),),
             "gate_up_proj": (("gate_proj", 0, inter), ("up_proj", inter, 2 * inter)), "down_proj": (("down_proj", 0, None),)}
    out = {}
    for name, t in adapters.items():
        if ".lora_A_" not in name:
            continue
        prefix, proj = name.split(".lora_A_")
        b = adapters[f"{prefix}.lora_B_{proj}"]
        for hf, lo, hi in split[proj]:
            base = f"base_model.model.model.{prefix}.{hf}"
            out[f"{base}.lora_A.weight"] = t.clone()
            out[f"{base}.lora_B.weight"] = b[lo:hi].clone()
    return out


def merge_lora_checkpoint(base_model: str, local_dir: str, target_dir: str, dtype=torch.bfloat16) -> dict:
    from safetensors.torch import save_file

    from verl_b200.models.config import PRESETS, ModelConfig
    from verl_b200.models.hf_io import load_hf_weights, save_hf_weights
    from verl_b200.models.lora import apply_lora, merged_hf_named_tensors
    from verl_b200.models.transformer import DecoderLM

    adapters, lcfg = _load_adapters(local_dir)
    if base_model in PRESETS:
        cfg = PRESETS[base_model]
        model = DecoderLM(cfg, dtype=dtype, seed=int(os.environ.get("VERL_B200_PRESET_SEED", "0")))
    else:
        cfg = ModelConfig.from_pretrained(base_model)
        model = DecoderLM(cfg, dtype=dtype, init=False)
        load_hf_weights(model, base_model)
    apply_lora(model, int(lcfg["rank"]), float(lcfg["alpha"]), list(lcfg["targets"]))
    own = dict(model.named_parameters())
    missing = [n for n in own if ".lora_" in n and n not in adapters]
    if missing:
        raise ValueError(f"the checkpoint lacks adapters for {missing[:3]} ...")
    with torch.no_grad():
        for n, t in adapters.items():
            own[n].copy_(t.to(own[n].dtype))
    os.makedirs(target_dir, exist_ok=True)
    cfg.save_pretrained(target_dir)
    save_hf_weights(merged_hf_named_tensors(model), target_dir)
    ad_dir = os.path.join(target_dir, "lora_adapter")
    os.makedirs(ad_dir, exist_ok=True)
    peft = _peft_tensors(cfg, {n: t.to(dtype) for n, t in adapters.items()})
    save_file(peft, os.path.join(ad_dir, "adapter_model.safetensors"))
    hf_targets = sorted({k.split(".")[-3] for k in peft})
    with open(os.path.join(ad_dir, "adapter_config.json"), "w") as f:
        json.dump({"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": int(lcfg["rank"]), "lora_alpha": float(lcfg["alpha"]), "lora_dropout": 0.0,
                   "bias": "none", "target_modules": hf_targets, "base_model_name_or_path": base_model}, f, indent=2)
    return {"merged": target_dir, "adapter": ad_dir, "num_adapter_tensors": len(peft)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--base_model", required=True, help="Hugging Face directory of the base model (or a preset name)")
    ap.add_argument("--local_dir", required=True, help="checkpoint directory of the LoRA run (…/global_step_N/actor)")
    ap.add_argument("--target_dir", required=True)
    a = ap.parse_args(argv)
    print(json.dumps(merge_lora_checkpoint(a.base_model, a.local_dir, a.target_dir)))


if __name__ == "__main__":
    main()
