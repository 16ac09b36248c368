"""Batch-container utilities of the engine path, on this framework's own ``TensorBatch`` / ``Jagged`` containers
(reference: ``verl/utils/tensordict_utils.py:26-813`` does the same on ``tensordict.TensorDict`` with nested tensors)."""

from __future__ import annotations

from typing import Any, Iterator, Optional, Sequence

import numpy as np
import torch

from verl_b200.protocol import DataProto, Jagged, TensorBatch

__all__ = ["get_tensordict", "assign_non_tensor", "get_non_tensor_data", "pop_non_tensor", "concat_jagged", "chunk_tensordict",
           "index_select_tensor_dict", "make_iterator", "pad_to_divisor", "unpad", "to_padded"]


def get_tensordict(tensors: dict[str, Any], non_tensors: Optional[dict] = None) -> DataProto:
    """Build a batch from a dict of tensors / lists (ragged lists of 1-D tensors become ``Jagged`` fields)."""
    fixed, extra = {}, dict(non_tensors or {})
    for k, v in tensors.items():
        if isinstance(v, torch.Tensor) or isinstance(v, Jagged):
            fixed[k] = v
        elif isinstance(v, (list, tuple)) and v and all(isinstance(x, torch.Tensor) for x in v):
            fixed[k] = Jagged.from_list(list(v)) if len({tuple(x.shape) for x in v}) > 1 else torch.stack(list(v))
        else:
            extra[k] = v
    n = len(next(iter(fixed.values()))) if fixed else None
    non_tensor, meta = {}, {}
    for k, v in extra.items():
        if isinstance(v, (list, tuple, np.ndarray)) and n is not None and len(v) == n:
            arr = np.empty(n, dtype=object)
            for i, x in enumerate(v):
                arr[i] = x
            non_tensor[k] = arr
        else:
            meta[k] = v
    return DataProto(batch=TensorBatch(fixed, batch_size=(n,)) if fixed else None, non_tensor_batch=non_tensor, meta_info=meta)


def assign_non_tensor(data: DataProto, **kwargs) -> DataProto:
    """Per-sample sequences go to ``non_tensor_batch``; everything else to ``meta_info``."""
    n = len(data)
    for k, v in kwargs.items():
        if isinstance(v, (list, tuple, np.ndarray)) and len(v) == n and n > 0:
            arr = np.empty(n, dtype=object)
            for i, x in enumerate(v):
                arr[i] = x
            data.non_tensor_batch[k] = arr
        else:
            data.meta_info[k] = v
    return data


def get_non_tensor_data(data: DataProto, key: str, default=None):
    if key in data.non_tensor_batch:
        return data.non_tensor_batch[key]
    return data.meta_info.get(key, default)


def pop_non_tensor(data: DataProto, key: str, default=None):
    if key in data.non_tensor_batch:
        return data.non_tensor_batch.pop(key)
    return data.meta_info.pop(key, default)


def concat_jagged(parts: Sequence[Jagged]) -> Jagged:
    rows = [r for p in parts for r in p.unbind()]
    return Jagged.from_list(rows)


def chunk_tensordict(data: DataProto, chunks: int) -> list[DataProto]:
    return data.chunk(chunks)


def index_select_tensor_dict(data: DataProto, indices) -> DataProto:
    idx = torch.as_tensor(indices, dtype=torch.int64)
    return data[idx]


def make_iterator(data: DataProto, mini_batch_size: int, epochs: int = 1, seed: Optional[int] = None) -> Iterator[DataProto]:
    return data.make_iterator(mini_batch_size, epochs, seed)


def pad_to_divisor(data: DataProto, divisor: int):
    from verl_b200.protocol import pad_dataproto_to_divisor

    return pad_dataproto_to_divisor(data, divisor)


def unpad(data: DataProto, pad_size: int) -> DataProto:
    return data[: len(data) - pad_size] if pad_size else data


def to_padded(j: Jagged, pad_value=0, max_len: Optional[int] = None, side: str = "right") -> torch.Tensor:
    rows = j.unbind()
    L = max_len or max((len(r) for r in rows), default=0)
    out = torch.full((len(rows), L, *rows[0].shape[1:]) if rows else (0, L), pad_value, dtype=rows[0].dtype if rows else torch.int64)
    for i, r in enumerate(rows):
        r = r[:L]
        if side == "right":
            out[i, : len(r)] = r
        else:
            out[i, L - len(r):] = r
    return out
