"""Batch-container utilities of the engine path, on this framework's own ``TensorBatch`` / ``Jagged`` containers
(reference: ``verl/utils/tensordict_utils.py:26-813`` does the same on ``tensordict.TensorDict`` with nested tensors)."""

from __future__ import annotations

from typing import Any, Iterator, Optional, Sequence

import numpy as np
import torch

from verl_b200.protocol import DataProto, Jagged, TensorBatch

__all__ = ["get_tensordict", "assign_non_tensor", "assign_non_tensor_data", "assign_non_tensor_stack", "unwrap_non_tensor_data",
           "get_non_tensor_data", "pop_non_tensor", "concat_jagged", "nested_tensor_from_tensor_list", "concat_nested_tensors",
           "concat_tensordict", "concat_tensordict_with_none_bsz", "chunk_tensordict", "index_select_tensor_dict", "union_tensor_dict",
           "make_iterator", "assert_tensordict_eq", "get", "get_keys", "pop", "pop_keys", "pad_to_divisor", "unpad", "contiguous",
           "maybe_fix_3d_position_ids", "list_of_dict_to_tensordict", "to_padded"]


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


# ---------------------------------------------------------------------------------------------------------------------
# The rest of the reference's helper surface (``verl/utils/tensordict_utils.py:26-950``) on these containers. A batch has three
# places for data: ``batch`` (tensors / Jagged rows, one entry per sample), ``non_tensor_batch`` (object arrays, one entry per
# sample) and ``meta_info`` (values shared by the whole batch) — the reference's NonTensorStack / NonTensorData distinction.
def assign_non_tensor_data(data: DataProto, key: str, val) -> DataProto:
    """One value for the whole batch."""
    data.meta_info[key] = val
    return data


def assign_non_tensor_stack(data: DataProto, key: str, val: Sequence) -> DataProto:
    """One value per sample (any Python objects, ragged lists included)."""
    if len(val) != len(data):
        raise ValueError(f"{key}: {len(val)} values for a batch of {len(data)}")
    arr = np.empty(len(val), dtype=object)
    for i, x in enumerate(val):
        arr[i] = x
    data.non_tensor_batch[key] = arr
    return data


def unwrap_non_tensor_data(x):
    """Plain Python view of a stored non-tensor value (object arrays become lists, 0-d arrays scalars)."""
    if isinstance(x, np.ndarray):
        return x.item() if x.ndim == 0 else x.tolist()
    return x


def nested_tensor_from_tensor_list(tensors: Sequence[torch.Tensor], ragged_idx: Optional[int] = None) -> Jagged:
    """Variable-length rows as one ``Jagged`` (the packed layout the varlen kernels consume)."""
    if ragged_idx not in (None, 0, 1):
        raise NotImplementedError("rows are ragged along their first dimension")
    return Jagged.from_list(list(tensors))


def concat_nested_tensors(tensors: Sequence[Jagged]) -> Jagged:
    return concat_jagged(tensors)


def concat_tensordict(data: Sequence[DataProto]) -> DataProto:
    """Samples of several batches behind one another; ``Jagged`` fields are concatenated row-wise, shared values must agree."""
    data = [d for d in data if d is not None]
    if not data:
        raise ValueError("nothing to concatenate")
    return DataProto.concat(list(data))


def concat_tensordict_with_none_bsz(data: Sequence[DataProto]) -> DataProto:
    """Batches that carry only shared values (no per-sample entries): the values of the first one win, later ones must not
    contradict them."""
    out = DataProto(batch=None, non_tensor_batch={}, meta_info={})
    for d in data:
        for k, v in d.meta_info.items():
            if k in out.meta_info and not _same(out.meta_info[k], v):
                raise ValueError(f"shared value {k!r} differs between the batches")
            out.meta_info.setdefault(k, v)
    return out


def union_tensor_dict(a: DataProto, b: DataProto) -> DataProto:
    """Fields of ``b`` added to ``a`` (same batch size; a field present in both must be equal)."""
    return a.union(b)


def _same(x, y) -> bool:
    if isinstance(x, torch.Tensor) or isinstance(y, torch.Tensor):
        return isinstance(x, torch.Tensor) and isinstance(y, torch.Tensor) and x.shape == y.shape and bool(torch.equal(x, y))
    if isinstance(x, Jagged) or isinstance(y, Jagged):
        return isinstance(x, Jagged) and isinstance(y, Jagged) and torch.equal(x.offsets, y.offsets) and torch.equal(x.values, y.values)
    if isinstance(x, np.ndarray) or isinstance(y, np.ndarray):
        xl, yl = unwrap_non_tensor_data(x), unwrap_non_tensor_data(y)
        return len(xl) == len(yl) and all(_same(p, q) for p, q in zip(xl, yl)) if isinstance(xl, list) and isinstance(yl, list) else xl == yl
    return x == y


def assert_tensordict_eq(a: DataProto, b: DataProto) -> None:
    ka, kb = (set(a.batch.keys()) if a.batch is not None else set()), (set(b.batch.keys()) if b.batch is not None else set())
    assert ka == kb, f"tensor keys differ: {sorted(ka ^ kb)}"
    for k in ka:
        assert _same(a.batch[k], b.batch[k]), f"tensor field {k!r} differs"
    assert set(a.non_tensor_batch) == set(b.non_tensor_batch), "per-sample non-tensor keys differ"
    for k in a.non_tensor_batch:
        assert _same(a.non_tensor_batch[k], b.non_tensor_batch[k]), f"non-tensor field {k!r} differs"
    assert set(a.meta_info) == set(b.meta_info), "shared keys differ"
    for k in a.meta_info:
        assert _same(a.meta_info[k], b.meta_info[k]), f"shared value {k!r} differs"


def get(data: DataProto, key: str, default=None):
    """Wherever the key lives: tensor field, per-sample objects (as a list) or shared value."""
    if data.batch is not None and key in data.batch.keys():
        return data.batch[key]
    if key in data.non_tensor_batch:
        return unwrap_non_tensor_data(data.non_tensor_batch[key])
    return data.meta_info.get(key, default)


def get_keys(data: DataProto, keys) -> DataProto:
    """A new batch holding only ``keys`` (from any of the three places); missing keys are an error."""
    keys = list(keys)
    t = {k: data.batch[k] for k in keys if data.batch is not None and k in data.batch.keys()}
    nt = {k: data.non_tensor_batch[k] for k in keys if k in data.non_tensor_batch}
    mi = {k: data.meta_info[k] for k in keys if k in data.meta_info}
    missing = [k for k in keys if k not in t and k not in nt and k not in mi]
    if missing:
        raise KeyError(f"keys {missing} not found")
    return DataProto(batch=TensorBatch(t, batch_size=(len(data),)) if t else None, non_tensor_batch=nt, meta_info=mi)


def pop(data: DataProto, key: str, default=None):
    if data.batch is not None and key in data.batch.keys():
        return data.batch.pop(key)
    if key in data.non_tensor_batch:
        return unwrap_non_tensor_data(data.non_tensor_batch.pop(key))
    return data.meta_info.pop(key, default)


def pop_keys(data: DataProto, keys) -> DataProto:
    out = get_keys(data, keys)
    for k in list(keys):
        pop(data, k)
    return out


def contiguous(data: DataProto) -> DataProto:
    if data.batch is not None:
        for k in list(data.batch.keys()):
            v = data.batch[k]
            data.batch[k] = Jagged(v.values.contiguous(), v.offsets) if isinstance(v, Jagged) else v.contiguous()
    return data


def maybe_fix_3d_position_ids(data: DataProto) -> DataProto:
    """Kept for call-site compatibility: the reference repairs the ragged index of nested 3-D position ids after a pickle round
    trip of its container; ``Jagged`` stores explicit offsets and survives pickling unchanged, so there is nothing to repair."""
    return data


def list_of_dict_to_tensordict(rows: Sequence[dict]) -> DataProto:
    """Rows of per-sample values → one batch (tensors of equal shape are stacked, ragged ones become ``Jagged``, everything
    else a per-sample object array)."""
    if not rows:
        raise ValueError("empty list")
    keys = list(rows[0])
    for r in rows:
        if list(r) != keys:
            raise ValueError("every row must carry the same keys")
    return get_tensordict({k: [r[k] for r in rows] for k in keys})
