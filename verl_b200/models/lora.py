"""Low-rank adapters on the decoder's projections.

``apply_lora(model, rank, alpha, target_modules)`` freezes every existing parameter and adds, per targeted projection
``W [out, in]``, trainable ``A [rank, in]`` (Kaiming-uniform) and ``B [out, rank]`` (zeros); the forward becomes
``x Wᵀ + (alpha / rank) · (x Aᵀ) Bᵀ``. Only the adapters enter the engine's flat parameter store, so optimizer state and
gradient collectives shrink to the adapter size. ``merged_hf_named_tensors`` yields HF-named tensors with the update
folded in — what the rollout replica and HF export need (reference: peft-based LoRA in the FSDP engine,
``verl/workers/engine/fsdp/transformer_impl.py`` ``lora_rank / lora_alpha / target_modules``; merge on weight sync).
"""

from __future__ import annotations

import math
from typing import Iterable, Iterator, Union

import torch
import torch.nn as nn

from verl_b200.models.transformer import DecoderLM, native_to_hf_tensors

__all__ = ["apply_lora", "lora_state_dict", "merged_hf_named_tensors", "merge_lora_", "TARGET_ALIASES"]

# HF module names → fused projections of this model
TARGET_ALIASES = {"q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj", "qkv_proj": "qkv_proj", "o_proj": "o_proj",
                  "gate_proj": "gate_up_proj", "up_proj": "gate_up_proj", "gate_up_proj": "gate_up_proj", "down_proj": "down_proj"}


def _targets(target_modules: Union[str, Iterable[str]]) -> set[str]:
    if target_modules in (None, "all-linear", "all"):
        return {"qkv_proj", "o_proj", "gate_up_proj", "down_proj"}
    names = [target_modules] if isinstance(target_modules, str) else list(target_modules)
    return {TARGET_ALIASES[n] for n in names}


def apply_lora(model: DecoderLM, rank: int = 16, alpha: float = 32.0, target_modules="all-linear", seed: int = 0) -> DecoderLM:
    assert rank > 0
    targets = _targets(target_modules)
    gen = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        p.requires_grad_(False)
    for layer in model.layers:
        for mod in (layer.self_attn, layer.mlp):
            adapters = {}
            for name in targets:
                w = getattr(mod, name, None)
                if not isinstance(w, nn.Parameter) or w.dim() != 2:
                    continue
                out_f, in_f = w.shape
                bound = 1.0 / math.sqrt(in_f)
                a = (torch.rand(rank, in_f, generator=gen) * 2 - 1) * bound * math.sqrt(3.0)
                mod.register_parameter(f"lora_A_{name}", nn.Parameter(a.to(dtype=w.dtype, device=w.device)))
                mod.register_parameter(f"lora_B_{name}", nn.Parameter(torch.zeros(out_f, rank, dtype=w.dtype, device=w.device)))
                adapters[name] = (f"lora_A_{name}", f"lora_B_{name}", alpha / rank)
            mod._lora = adapters
    model.lora_config = {"rank": rank, "alpha": alpha, "targets": sorted(targets)}
    return model


def lora_state_dict(model: DecoderLM) -> dict[str, torch.Tensor]:
    return {n: p.detach() for n, p in model.named_parameters() if ".lora_A_" in n or ".lora_B_" in n}


def _merged_params(model: DecoderLM) -> dict[str, torch.Tensor]:
    params = {n: p for n, p in model.named_parameters() if ".lora_" not in n}
    for li, layer in enumerate(model.layers):
        for prefix, mod in ((f"layers.{li}.self_attn.", layer.self_attn), (f"layers.{li}.mlp.", layer.mlp)):
            for name, (a, b, scale) in (getattr(mod, "_lora", None) or {}).items():
                w = params[prefix + name]
                delta = (getattr(mod, b).float() @ getattr(mod, a).float()) * scale
                params[prefix + name] = (w.float() + delta).to(w.dtype)
    return params


def merged_hf_named_tensors(model: DecoderLM) -> Iterator[tuple[str, torch.Tensor]]:
    return native_to_hf_tensors(model.cfg, _merged_params(model))


@torch.no_grad()
def merge_lora_(model: DecoderLM) -> DecoderLM:
    """Fold the adapters into the base weights in place and remove them (export of a fine-tuned model)."""
    merged = _merged_params(model)
    own = dict(model.named_parameters())
    for n, t in merged.items():
        own[n].copy_(t)
    for layer in model.layers:
        for mod in (layer.self_attn, layer.mlp):
            for name, (a, b, _) in (getattr(mod, "_lora", None) or {}).items():
                delattr(mod, a)
                delattr(mod, b)
            mod._lora = None
    return model
