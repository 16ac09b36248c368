"""Compatibility gates for the HuggingFace ecosystem (reference: ``verl/utils/transformers_compat.py:40-95``): version
checks and the tied-weights key handling used when exporting / importing checkpoints."""

from __future__ import annotations

from functools import lru_cache

from packaging import version

__all__ = ["transformers_version", "is_transformers_version_in_range", "drop_tied_weight_keys", "flash_attn_available"]


@lru_cache
def transformers_version():
    try:
        import transformers

        return version.parse(transformers.__version__)
    except ImportError:
        return None


def is_transformers_version_in_range(min_version: str = None, max_version: str = None) -> bool:
    v = transformers_version()
    if v is None:
        return False
    if min_version is not None and v < version.parse(min_version):
        return False
    if max_version is not None and v > version.parse(max_version):
        return False
    return True


def drop_tied_weight_keys(state_dict: dict, tie_word_embeddings: bool) -> dict:
    """HF checkpoints of tied models must not carry ``lm_head.weight`` (transformers ≥ 4.5x warns or fails on load)."""
    if tie_word_embeddings and "lm_head.weight" in state_dict:
        state_dict = dict(state_dict)
        state_dict.pop("lm_head.weight")
    return state_dict


def flash_attn_available() -> bool:
    """Always False for dispatch purposes: attention runs on this framework's own kernels."""
    return False
