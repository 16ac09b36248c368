"""Names ↔ torch dtypes (reference: ``verl/utils/torch_dtypes.py:25`` ``PrecisionType``)."""

from __future__ import annotations

import torch

__all__ = ["PrecisionType"]

_HALF = ("fp16", "16", "half", "float16", torch.float16)
_FULL = ("fp32", "32", "float", "float32", torch.float32)
_BF16 = ("bf16", "bfloat16", torch.bfloat16)


class PrecisionType:
    @staticmethod
    def is_fp16(p) -> bool:
        return p in _HALF

    @staticmethod
    def is_fp32(p) -> bool:
        return p in _FULL

    @staticmethod
    def is_bf16(p) -> bool:
        return p in _BF16

    @staticmethod
    def to_dtype(p) -> torch.dtype:
        if p in _HALF:
            return torch.float16
        if p in _FULL:
            return torch.float32
        if p in _BF16:
            return torch.bfloat16
        raise RuntimeError(f"unexpected precision: {p}")

    @staticmethod
    def to_str(p: torch.dtype) -> str:
        return {torch.float16: "fp16", torch.float32: "fp32", torch.bfloat16: "bf16"}[p]
