"""Analytic FLOPs estimate → MFU.

Every architecture is reduced to one :class:`ArchCost` — weights each token multiplies against (so ``6 · N`` FLOPs per
token for forward + backward), plus the attention score / value products, which scale with ``Σ L · span(L)`` per layer —
and one generic formula evaluates it. Families (keyed by ``model_type``): dense Llama / Qwen2 / Qwen3 / Mistral style,
routed mixture-of-experts with optional shared experts, DeepSeek-V3 (MLA projections, leading dense layers), Gemma-3 and
GPT-OSS (sliding-window layers), Qwen3.5 (gated-delta linear-attention layers + gated full attention), Apertus
(non-gated MLP), and the Qwen-VL variants (language model + vision tower on ``images_seqlens``).

Parity target: ``verl/utils/flops_counter.py`` (device peaks :22-44, per-architecture estimators :92-704, ``FlopsCounter``
:704-746). Conventions kept from there so that MFU numbers are comparable: the embedding and the output matrix count as
``2 · V · H`` weights, full attention costs ``12 · L² · d · heads`` per layer for forward + backward (``6`` where the
reference counts the causal half: DeepSeek-V3, Gemma-3, Qwen3.5, GPT-OSS), a forward-only pass is reported as ``/ 3`` by
the caller.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence

import torch

__all__ = ["FlopsCounter", "ArchCost", "get_device_flops", "DEVICE_PEAK_FLOPS", "register_arch", "arch_cost"]

# dense bf16 peak per device name fragment (first match wins, so more specific names come first)
DEVICE_PEAK_FLOPS = {"GB200": 2.5e15, "B200": 2.25e15, "MI355X": 2500e12, "MI350X": 2300e12, "MI300X": 1307e12, "H100": 989e12,
                     "H800": 989e12, "H200": 989e12, "H20": 148e12, "A100": 312e12, "A800": 312e12, "L40S": 362.05e12, "L40": 181.05e12,
                     "A40": 149.7e12, "L20": 119.5e12, "RTX 3070 Ti": 21.75e12, "CPU": 448e9}


def get_device_flops(unit: str = "T", device_name: Optional[str] = None) -> float:
    """Peak dense bf16 FLOP/s of the current (or named) device in the given unit; ``inf`` for unknown devices."""
    name = device_name or (torch.cuda.get_device_name() if torch.cuda.is_available() else "CPU")
    flops = float("inf")
    for key, val in DEVICE_PEAK_FLOPS.items():
        if key in name:
            flops = val
            break
    return flops / {"B": 1e9, "K": 1e3, "M": 1e6, "G": 1e9, "T": 1e12, "P": 1e15}[unit]


def _get(cfg: Any, name: str, default=None):
    if isinstance(cfg, dict):
        v = cfg.get(name, default)
    else:
        v = getattr(cfg, name, default)
        if v is None and hasattr(cfg, "extra") and isinstance(getattr(cfg, "extra"), dict):
            v = cfg.extra.get(name, default)
    return default if v is None else v


@dataclass
class ArchCost:
    """What one token costs. ``layer_weights[i]``: matrix elements layer ``i`` multiplies a token against;
    ``other_weights``: embedding + output matrix (and anything else outside the layers); ``attn_layers``: per layer
    ``(qk_dim + v_dim) · heads`` and a span function ``L → keys seen`` (``None`` = no softmax attention);
    ``attn_factor``: 6 for a full (non-causal) count of forward + backward, 3 for the causal half;
    ``per_token_extra``: FLOPs per token that are not matrix weights (recurrences)."""

    layer_weights: list = field(default_factory=list)
    other_weights: float = 0.0
    attn_layers: list = field(default_factory=list)        # [(dims_times_heads, span_fn or None)]
    attn_factor: float = 6.0
    per_token_extra: float = 0.0
    vision: Optional[Any] = None                            # vision tower config (costed on images_seqlens)

    def flops(self, batch_seqlens: Sequence[int], images_seqlens: Optional[Sequence[int]] = None) -> float:
        tokens = float(sum(batch_seqlens))
        total = 6.0 * (sum(self.layer_weights) + self.other_weights) * tokens + self.per_token_extra * tokens
        for dims, span in self.attn_layers:
            if span is None:
                continue
            total += self.attn_factor * dims * sum(float(L) * float(span(L)) for L in batch_seqlens)
        if self.vision is not None and images_seqlens is not None:
            total += _vision_tower_flops(self.vision, images_seqlens)
        return total


_ARCH: dict[str, Callable[[Any], ArchCost]] = {}


def register_arch(*names: str):
    def deco(fn):
        for n in names:
            _ARCH[n] = fn
        return fn

    return deco


def _dims(c):
    h = _get(c, "hidden_size")
    nh, nkv = _get(c, "num_attention_heads"), _get(c, "num_key_value_heads", _get(c, "num_attention_heads"))
    d = _get(c, "head_dim", h // nh)
    return h, nh, nkv, d


def _full(L):
    return L


@register_arch("qwen2", "llama", "qwen3", "mistral", "minicpmv", "minicpmo", "seed_oss", "glm4", "internlm2")
def _dense(c, mlp_mats: int = 3) -> ArchCost:
    h, nh, nkv, d = _dims(c)
    n = _get(c, "num_hidden_layers")
    attn = h * (nh * d + 2 * nkv * d) + nh * d * h
    mlp = mlp_mats * h * _get(c, "intermediate_size")
    return ArchCost([attn + mlp] * n, 2.0 * _get(c, "vocab_size") * h, [((d + d) * nh, _full)] * n, 6.0)


@register_arch("apertus")
def _apertus(c) -> ArchCost:
    return _dense(c, mlp_mats=2)        # xIELU MLP: up and down projections only


@register_arch("qwen2_moe", "qwen3_moe")
def _routed_moe(c) -> ArchCost:
    h, nh, nkv, d = _dims(c)
    n = _get(c, "num_hidden_layers")
    attn = h * (nh * d + 2 * nkv * d) + nh * d * h
    topk, e = _get(c, "num_experts_per_tok"), _get(c, "num_experts", _get(c, "n_routed_experts", 0))
    mlp = 3 * h * _get(c, "moe_intermediate_size") * topk + h * e
    shared = _get(c, "shared_expert_intermediate_size", 0)
    if shared:
        mlp += 3 * h * shared + h
    return ArchCost([attn + mlp] * n, 2.0 * _get(c, "vocab_size") * h, [((d + d) * nh, _full)] * n, 6.0)


@register_arch("deepseek_v3", "deepseek_v2", "kimi_k2")
def _deepseek_v3(c) -> ArchCost:
    h, nh = _get(c, "hidden_size"), _get(c, "num_attention_heads")
    n, dense_first = _get(c, "num_hidden_layers"), _get(c, "first_k_dense_replace", 0)
    qk_nope, qk_rope, dv, kv_rank = _get(c, "qk_nope_head_dim"), _get(c, "qk_rope_head_dim"), _get(c, "v_head_dim"), _get(c, "kv_lora_rank")
    dq = qk_nope + qk_rope
    q_rank = _get(c, "q_lora_rank", 0)
    attn = (h * q_rank + q_rank * nh * dq) if q_rank else h * nh * dq           # (low-rank) query projection
    attn += h * (kv_rank + qk_rope)                                              # compressed KV + shared rope key
    attn += nh * (qk_nope + dv) * kv_rank                                        # up-projection of keys and values
    attn += nh * dv * h                                                          # output projection
    moe = h * _get(c, "n_routed_experts") + 3 * h * _get(c, "moe_intermediate_size") * (_get(c, "num_experts_per_tok") + _get(c, "n_shared_experts", 0))
    dense = 3 * h * _get(c, "intermediate_size")
    layers = [attn + (dense if i < dense_first else moe) for i in range(n)]
    return ArchCost(layers, 2.0 * _get(c, "vocab_size") * h, [((dq + dv) * nh, _full)] * n, 3.0)


def _layer_types(c, n: int, default_pattern: int) -> list:
    lt = _get(c, "layer_types", None)
    if lt:
        return list(lt)
    pat = _get(c, "sliding_window_pattern", default_pattern)
    return ["sliding_attention" if (i + 1) % pat else "full_attention" for i in range(n)]


@register_arch("gemma3_text", "gemma3", "gemma2")
def _gemma3(c) -> ArchCost:
    base = _dense(c)
    h, nh, nkv, d = _dims(c)
    n = _get(c, "num_hidden_layers")
    win = _get(c, "sliding_window", 1024)
    spans = [(lambda L, w=win: min(L, w)) if t == "sliding_attention" and win else _full for t in _layer_types(c, n, 6)]
    return ArchCost(base.layer_weights, base.other_weights, [((d + d) * nh, s) for s in spans], 3.0)


@register_arch("gpt_oss")
def _gpt_oss(c) -> ArchCost:
    h, nh, nkv, d = _dims(c)
    n = _get(c, "num_hidden_layers")
    attn = h * (nh * d + 2 * nkv * d) + nh * d * h
    e, topk = _get(c, "num_local_experts", _get(c, "num_experts", 0)), _get(c, "num_experts_per_tok", _get(c, "experts_per_token", 0))
    mlp = 3 * h * _get(c, "intermediate_size") * topk + h * e
    win = _get(c, "sliding_window", 128)
    spans = [(lambda L, w=win: min(L, w)) if t == "sliding_attention" and win else _full for t in _layer_types(c, n, 2)]
    return ArchCost([attn + mlp] * n, 2.0 * _get(c, "vocab_size") * h, [((d + d) * nh, s) for s in spans], 3.0)


@register_arch("qwen3_5", "qwen3_5_moe", "qwen3_next")
def _qwen3_5(c) -> ArchCost:
    vis = _get(c, "vision_config", None)
    c = _get(c, "text_config", c)
    h, nh, nkv, d = _dims(c)
    n = _get(c, "num_hidden_layers")
    lt = _get(c, "layer_types", None) or ["linear_attention" if (i + 1) % _get(c, "full_attention_interval", 4) else "full_attention" for i in range(n)]
    # full-attention layers: the query projection also emits a sigmoid gate (2x), plus k, v and the output projection
    full_attn = h * (2 * nh * d + 2 * nkv * d + nh * d)
    lk = _get(c, "linear_num_key_heads", 0) * _get(c, "linear_key_head_dim", 0)
    lv = _get(c, "linear_num_value_heads", 0) * _get(c, "linear_value_head_dim", 0)
    lin_attn = h * (2 * lk + 3 * lv + 2 * _get(c, "linear_num_value_heads", 0)) + _get(c, "linear_conv_kernel_dim", 0) * (2 * lk + lv)
    if _get(c, "num_experts", 0):
        mlp = h * _get(c, "num_experts") + 3 * h * _get(c, "moe_intermediate_size") * _get(c, "num_experts_per_tok")
        mlp += 3 * h * _get(c, "shared_expert_intermediate_size", 0) + h
    else:
        mlp = 3 * h * _get(c, "intermediate_size")
    layers = [(full_attn if t == "full_attention" else lin_attn) + mlp for t in lt]
    n_lin = sum(t != "full_attention" for t in lt)
    # gated delta rule: state update and read-out per token, per value head (forward + backward)
    recur = 15.0 * _get(c, "linear_key_head_dim", 0) * _get(c, "linear_value_head_dim", 0) * _get(c, "linear_num_value_heads", 0) * n_lin
    return ArchCost(layers, 2.0 * _get(c, "vocab_size") * h, [((d + d) * nh, _full if t == "full_attention" else None) for t in lt], 3.0,
                    per_token_extra=recur, vision=vis)


@register_arch("qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "glm4v", "kimi_vl")
def _qwen_vl(c) -> ArchCost:
    vis = _get(c, "vision_config", _get(c, "vision", None))
    text = _get(c, "text_config", c)
    base = _routed_moe(text) if _get(text, "num_experts", 0) else _dense(text)
    base.vision = vis
    return base


def _vision_tower_flops(v, images_seqlens: Sequence[int]) -> float:
    """ViT on ``images_seqlens`` patch tokens per image: patch embedding, ``depth`` blocks (full attention), patch merger(s)."""
    dim = _get(v, "hidden_size", _get(v, "embed_dim"))
    heads, depth = _get(v, "num_heads"), _get(v, "depth")
    mlp_hidden = _get(v, "intermediate_size", int(dim * float(_get(v, "mlp_ratio", 4.0))))
    merge = _get(v, "spatial_merge_size", 2) ** 2
    out_dim = _get(v, "out_hidden_size", _get(v, "hidden_size", dim))
    patch = dim * _get(v, "in_channels", 3) * _get(v, "temporal_patch_size", 2) * _get(v, "patch_size", 14) ** 2
    gated = bool(_get(v, "gated_mlp", _get(v, "hidden_act", "") == "silu"))
    block = dim * 4 * dim + (3 if gated else 2) * dim * mlp_hidden
    merger = (out_dim + dim * merge) * (dim * merge)
    n_merger = 1 + len(_get(v, "deepstack_visual_indexes", []) or [])
    tokens = float(sum(images_seqlens))
    dense = 6.0 * (patch + block * depth + merger * n_merger) * tokens
    attn = 12.0 * sum(float(L) * float(L) for L in images_seqlens) * (dim // heads) * heads * depth
    return dense + attn


def arch_cost(config) -> ArchCost:
    mt = str(_get(config, "model_type", "qwen2"))
    fn = _ARCH.get(mt)
    if fn is None:
        # unknown types: mixture-of-experts fields → routed-MoE formula, else dense (the reference reports 0 for unknown types)
        fn = _routed_moe if _get(config, "num_experts", 0) and _get(config, "moe_intermediate_size", 0) else _dense
    return fn(config)


class FlopsCounter:
    """``estimate_flops(batch_seqlens, delta_time)`` → (achieved TFLOP/s for forward + backward, device peak TFLOP/s)."""

    def __init__(self, config):
        self.config = config
        self.cost = arch_cost(config)

    def estimate_flops(self, batch_seqlens, delta_time: float, **kwargs):
        fl = self.cost.flops(list(batch_seqlens), kwargs.get("images_seqlens"))
        return fl / max(delta_time, 1e-9) / 1e12, get_device_flops("T")
