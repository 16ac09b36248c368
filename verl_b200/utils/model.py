"""Model-level helpers (reference: ``verl/utils/model.py``): config loading, random masks for tests, value-head
construction, parameter counting and size reports."""

from __future__ import annotations

import json
import os
from typing import Optional

import torch

from verl_b200.models.config import PRESETS, ModelConfig
from verl_b200.models.transformer import DecoderLM
from verl_b200.utils.torch_functional import compute_position_id_with_mask

__all__ = ["get_model_config", "get_generation_config", "create_random_mask", "compute_position_id_with_mask", "create_actor_model",
           "create_critic_model", "load_valuehead_model", "get_model_size", "print_model_size", "update_model_config"]


def get_model_config(path_or_preset: str, override: Optional[dict] = None) -> ModelConfig:
    cfg = PRESETS[path_or_preset] if path_or_preset in PRESETS else ModelConfig.from_pretrained(os.path.expanduser(path_or_preset))
    return update_model_config(cfg, override or {})


def update_model_config(cfg: ModelConfig, override: dict) -> ModelConfig:
    known = {k: v for k, v in dict(override).items() if k in ModelConfig.__dataclass_fields__}
    return cfg.replace(**known) if known else cfg


def get_generation_config(path: str) -> Optional[dict]:
    f = os.path.join(os.path.expanduser(path), "generation_config.json")
    return json.load(open(f)) if os.path.exists(f) else None


def create_random_mask(input_ids: torch.Tensor, max_ratio_of_valid_token: float, max_ratio_of_left_padding: float,
                       min_ratio_of_valid_token: float = 0.0) -> torch.Tensor:
    """Left padding followed by a run of valid tokens followed by right padding, per row (test fixture)."""
    assert 0 < max_ratio_of_valid_token <= 1 and 0 <= max_ratio_of_left_padding < 1
    B, S = input_ids.shape
    mask = torch.zeros(B, S, dtype=torch.int64)
    for i in range(B):
        left = int(torch.randint(0, int(S * max_ratio_of_left_padding) + 1, (1,)))
        lo = max(1, int(S * min_ratio_of_valid_token))
        hi = max(lo, min(int(S * max_ratio_of_valid_token), S - left))
        n = int(torch.randint(lo, hi + 1, (1,)))
        mask[i, left: left + n] = 1
    return mask


def create_actor_model(path_or_preset: str, dtype=torch.bfloat16, device="cpu", override: Optional[dict] = None, seed: int = 0) -> DecoderLM:
    cfg = get_model_config(path_or_preset, override)
    model = DecoderLM(cfg, dtype=dtype, device=device, init=True, seed=seed)
    if path_or_preset not in PRESETS:
        from verl_b200.models.hf_io import load_hf_weights

        load_hf_weights(model, os.path.expanduser(path_or_preset))
    return model


def load_valuehead_model(path_or_preset: str, dtype=torch.bfloat16, device="cpu", override: Optional[dict] = None, seed: int = 0) -> DecoderLM:
    """Trunk from the checkpoint, scalar head from ``score.weight`` when the checkpoint has one (token-classification
    export) and freshly initialised otherwise."""
    cfg = get_model_config(path_or_preset, override).replace(value_head=True)
    model = DecoderLM(cfg, dtype=dtype, device=device, init=True, seed=seed)
    if path_or_preset not in PRESETS:
        from verl_b200.models.hf_io import load_hf_weights

        load_hf_weights(model, os.path.expanduser(path_or_preset), strict=False)
    return model


create_critic_model = load_valuehead_model


def get_model_size(model: torch.nn.Module, scale: str = "auto") -> tuple[float, str]:
    n = sum(p.numel() for p in model.parameters())
    if scale == "auto":
        scale = "B" if n > 1e9 else "M" if n > 1e6 else "K" if n > 1e3 else ""
    div = {"B": 1e9, "M": 1e6, "K": 1e3, "": 1}[scale]
    return n / div, scale


def print_model_size(model: torch.nn.Module, name: Optional[str] = None):
    n, s = get_model_size(model)
    print(f"{name or type(model).__name__} contains {n:.2f}{s} parameters")
