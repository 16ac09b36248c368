"""Analytic FLOPs estimate → MFU. Parity target: ``verl/utils/flops_counter.py`` (device peaks :22-44,
per-architecture formulas :92-704): dense ``6·N·T + 12·Σ L²·d_head·n_head·layers`` (fwd+bwd), MoE counts active
experts only."""

from __future__ import annotations

import torch

from verl_b200.models.config import ModelConfig

__all__ = ["FlopsCounter", "get_device_flops", "DEVICE_PEAK_FLOPS"]

# dense bf16 peak per device (same table values as the reference for the entries that matter here)
DEVICE_PEAK_FLOPS = {"B200": 2.25e15, "GB200": 2.5e15, "H100": 989e12, "H800": 989e12, "H200": 989e12, "H20": 148e12,
                     "A100": 312e12, "A800": 312e12, "L40": 181.05e12, "L20": 119.5e12, "CPU": 448e9}


def get_device_flops(unit: str = "T") -> float:
    name = torch.cuda.get_device_name() if torch.cuda.is_available() else "CPU"
    flops = float("inf")
    for key, val in DEVICE_PEAK_FLOPS.items():
        if key in name:
            flops = val
            break
    div = {"B": 1e9, "K": 1e3, "M": 1e6, "G": 1e9, "T": 1e12, "P": 1e15}[unit]
    return flops / div


class FlopsCounter:
    def __init__(self, config: ModelConfig):
        self.config = config

    def _dense_params_per_token(self) -> float:
        c = self.config
        h = c.hidden_size
        attn = h * (c.q_size + 2 * c.kv_size) + c.q_size * h
        if c.is_moe:
            mlp = c.num_experts_per_tok * 3 * h * c.moe_intermediate_size + h * c.num_experts
        else:
            mlp = 3 * h * c.intermediate_size
        emb = c.vocab_size * h  # lm_head (the embedding lookup costs no FLOPs)
        return c.num_hidden_layers * (attn + mlp) + emb

    def estimate_flops(self, batch_seqlens, delta_time: float):
        """Returns (achieved TFLOP/s, device peak TFLOP/s) for one forward+backward over the given sequences."""
        c = self.config
        tokens = float(sum(batch_seqlens))
        seqlen_sq = float(sum(float(s) * float(s) for s in batch_seqlens))
        dense = 6.0 * self._dense_params_per_token() * tokens
        attn = 12.0 * seqlen_sq * c.head_dim * c.num_attention_heads * c.num_hidden_layers
        achieved = (dense + attn) / max(delta_time, 1e-9) / 1e12
        return achieved, get_device_flops("T")
