"""Splitting a ``DecoderLM`` over tensor-parallel ranks and pipeline stages, and putting it back together.

Layout rules (Megatron-style; the reference obtains them from Megatron-Bridge, ``verl/workers/engine/megatron/
transformer_impl.py:324-360`` and ``verl/models/mcore/*``):

* ``embed_tokens`` / ``lm_head``      rows (vocabulary) split evenly;
* ``qkv_proj`` / ``qkv_bias``          each of the q | k | v row blocks split by heads, the local tensor is [q_r | k_r | v_r];
* ``o_proj`` / ``down_proj``           columns (input features) split;
* ``gate_up_proj``                      each of the gate | up row blocks split, local tensor [gate_r | up_r];
* MoE ``experts_gate_up`` / ``experts_down``: the same per expert (expert tensor parallelism);
* norms, router, value head            replicated.

Pipeline stages own contiguous layer ranges; stage 0 additionally the embedding, the last stage final norm + head.
"""

from __future__ import annotations

from typing import Optional

import torch

from verl_b200.models.config import ModelConfig

__all__ = ["local_model_config", "stage_layer_range", "shard_param", "unshard_param", "local_to_global_name", "tp_rule",
           "build_rollout_shard", "refresh_rollout_shard", "VisionLanguageRolloutShard"]


def local_model_config(cfg: ModelConfig, tp: int, shard_vocab: bool = True) -> ModelConfig:
    if tp == 1:
        return cfg
    assert cfg.num_attention_heads % tp == 0 and cfg.num_key_value_heads % tp == 0, "head counts must divide by the TP size"
    assert (cfg.vocab_size % tp == 0 or not shard_vocab) and cfg.intermediate_size % tp == 0
    kw = dict(num_attention_heads=cfg.num_attention_heads // tp, num_key_value_heads=cfg.num_key_value_heads // tp,
              intermediate_size=cfg.intermediate_size // tp, vocab_size=cfg.vocab_size // tp if shard_vocab else cfg.vocab_size,
              head_dim=cfg.head_dim)
    if cfg.is_moe:
        assert cfg.moe_intermediate_size % tp == 0
        kw["moe_intermediate_size"] = cfg.moe_intermediate_size // tp
    return cfg.replace(**kw)


def stage_layer_range(num_layers: int, pp: int, stage: int) -> range:
    """Contiguous split; the first ``num_layers % pp`` stages get one extra layer."""
    base, extra = divmod(num_layers, pp)
    start = stage * base + min(stage, extra)
    return range(start, start + base + (1 if stage < extra else 0))


def tp_rule(name: str, cfg: ModelConfig):
    """(dim, segments) for a parameter name of the FULL model; ``None`` when replicated. ``segments`` lists the sizes of
    the row/column blocks that are split independently (one block = plain split)."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf in ("embed_tokens", "lm_head"):
        return 0, [cfg.vocab_size]
    if leaf in ("qkv_proj", "qkv_bias"):
        return 0, [cfg.q_size, cfg.kv_size, cfg.kv_size]
    if leaf == "o_proj":
        return 1, [cfg.q_size]
    if leaf == "gate_up_proj":
        return 0, [cfg.intermediate_size, cfg.intermediate_size]
    if leaf == "up_proj":
        return 0, [cfg.intermediate_size]
    if leaf == "down_proj":
        return 1, [cfg.intermediate_size]
    if leaf == "experts_gate_up":
        return 1, [cfg.moe_intermediate_size, cfg.moe_intermediate_size]
    if leaf == "experts_down":
        return 2, [cfg.moe_intermediate_size]
    return None


def shard_param(name: str, full: torch.Tensor, cfg: ModelConfig, tp_rank: int, tp: int) -> torch.Tensor:
    rule = tp_rule(name, cfg)
    if rule is None or tp == 1:
        return full
    dim, segs = rule
    parts, off = [], 0
    for n in segs:
        per = n // tp
        parts.append(full.narrow(dim, off + tp_rank * per, per))
        off += n
    return parts[0] if len(parts) == 1 else torch.cat(parts, dim)


def unshard_param(name: str, shards: list[torch.Tensor], cfg: ModelConfig) -> torch.Tensor:
    """Inverse of :func:`shard_param`; ``cfg`` is the FULL model's config, ``shards`` are ordered by TP rank."""
    rule = tp_rule(name, cfg)
    tp = len(shards)
    if rule is None or tp == 1:
        return shards[0]
    dim, segs = rule
    out, off = [], 0
    for n in segs:
        per = n // tp
        out.extend(s.narrow(dim, off, per) for s in shards)
        off += per
    return torch.cat(out, dim)


def local_to_global_name(name: str, layer_offset: int) -> str:
    if name.startswith("layers.") and layer_offset:
        _, idx, rest = name.split(".", 2)
        return f"layers.{int(idx) + layer_offset}.{rest}"
    return name


def build_rollout_shard(full, tp_rank: int, tp: int):
    """Tensor-parallel slice of ``full`` for the rollout engine: decoder layers are cut like in training (copies), while
    embedding, final norm and output matrix stay whole and SHARE the trainer's storage (the sampler wants full logits on
    every rank, and those tensors are read-only here)."""
    import torch

    from verl_b200.models.transformer import DecoderLM

    cfg = full.cfg
    local = DecoderLM(local_model_config(cfg, tp, shard_vocab=False), dtype=full.dtype, device=full.embed_tokens.device, init=False)
    local.embed_tokens = full.embed_tokens
    local.norm = full.norm
    if full.lm_head is not None:
        local.lm_head = full.lm_head
    refresh_rollout_shard(local, full, tp_rank, tp)
    return local


class VisionLanguageRolloutShard(torch.nn.Module):
    """What a tensor-parallel rollout replica holds of a vision-language model: its slice of the decoder, and the vision tower
    whole and shared with the trainer (every rank of the replica embeds the same images and gets the same rows, so nothing has to
    be exchanged; the tower is a few percent of the model)."""

    def __init__(self, full_vl, tp_rank: int, tp: int):
        super().__init__()
        self.visual, self.vcfg = full_vl.visual, full_vl.vcfg
        self.language_model = build_rollout_shard(full_vl.language_model, tp_rank, tp)
        self.cfg = self.language_model.cfg


def refresh_rollout_shard(local, full, tp_rank: int, tp: int) -> None:
    """Re-cut the layer shards after the trainer's weights changed (one device-to-device copy of 1/tp of the layers)."""
    import torch

    src = dict(full.named_parameters())
    with torch.no_grad():
        for name, p in local.named_parameters():
            if name.startswith("layers."):
                p.copy_(shard_param(name, src[name], full.cfg, tp_rank, tp))
