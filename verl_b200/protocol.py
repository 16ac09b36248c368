"""Batch protocol exchanged between the controller and workers.

``DataProto`` bundles a dictionary of tensors that share a leading batch dimension (``batch``), a dictionary of
``numpy`` object arrays of the same length (``non_tensor_batch``) and free-form ``meta_info``. It offers the
operations the PPO/GRPO dataflows need: select / pop / union / chunk / split / concat / repeat / reorder / slicing /
padding to a divisor / mini-batch iteration / (de)serialisation.

Behavioural parity target: ``verl/protocol.py`` (DataProto at :318, pad helpers at :74, chunk :861, concat :914,
repeat :968, DataProtoFuture :1171, all_gather_data_proto :1331). The tensor container is an in-house ``TensorBatch``
instead of ``tensordict.TensorDict`` and supports jagged (nested) entries through :class:`Jagged`.
"""

from __future__ import annotations

import copy
import io
import math
import os
import pickle
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator, Optional, Sequence, Union

import numpy as np
import torch

__all__ = [
    "Jagged",
    "TensorBatch",
    "DataProto",
    "DataProtoItem",
    "DataProtoFuture",
    "pad_dataproto_to_divisor",
    "unpad_dataproto",
    "union_tensor_dict",
    "union_numpy_dict",
    "collate_fn",
    "all_gather_data_proto",
]


# --------------------------------------------------------------------------------------------------------------
# Jagged tensor: values [total, ...] + offsets [B+1]. Replaces torch nested tensors in the engine path.
# --------------------------------------------------------------------------------------------------------------
class Jagged:
    """A batch of variable-length rows stored back to back (the layout packed-varlen kernels consume)."""

    __slots__ = ("values", "offsets")

    def __init__(self, values: torch.Tensor, offsets: torch.Tensor):
        assert offsets.dim() == 1 and offsets.numel() >= 1
        self.values = values
        self.offsets = offsets.to(torch.int64)

    @classmethod
    def from_list(cls, rows: Sequence[torch.Tensor]) -> "Jagged":
        lens = torch.tensor([0] + [int(r.shape[0]) for r in rows], dtype=torch.int64)
        values = torch.cat(list(rows), dim=0) if len(rows) else torch.empty(0)
        return cls(values, torch.cumsum(lens, 0))

    @classmethod
    def from_padded(cls, padded: torch.Tensor, lengths: torch.Tensor, left_pad: bool = False) -> "Jagged":
        B, L = padded.shape[:2]
        idx = torch.arange(L, device=padded.device)[None, :]
        lengths = lengths.to(padded.device)
        mask = idx >= (L - lengths[:, None]) if left_pad else idx < lengths[:, None]
        offsets = torch.zeros(B + 1, dtype=torch.int64, device=padded.device)
        offsets[1:] = torch.cumsum(lengths, 0)
        return cls(padded[mask], offsets)

    def __len__(self) -> int:
        return self.offsets.numel() - 1

    @property
    def lengths(self) -> torch.Tensor:
        return self.offsets[1:] - self.offsets[:-1]

    @property
    def device(self):
        return self.values.device

    def row(self, i: int) -> torch.Tensor:
        return self.values[int(self.offsets[i]) : int(self.offsets[i + 1])]

    def unbind(self) -> list[torch.Tensor]:
        return [self.row(i) for i in range(len(self))]

    def to(self, *args, **kwargs) -> "Jagged":
        return Jagged(self.values.to(*args, **kwargs), self.offsets.to(kwargs.get("device", args[0] if args and not isinstance(args[0], torch.dtype) else self.offsets.device)))

    def index(self, idx: torch.Tensor) -> "Jagged":
        rows = self.unbind()
        return Jagged.from_list([rows[int(i)] for i in idx.tolist()]) if len(idx) else Jagged(self.values[:0], self.offsets[:1])

    def slice(self, start: int, stop: int) -> "Jagged":
        s, e = int(self.offsets[start]), int(self.offsets[stop])
        return Jagged(self.values[s:e], self.offsets[start : stop + 1] - self.offsets[start])

    def to_padded(self, pad_value=0, max_len: Optional[int] = None) -> torch.Tensor:
        lens = self.lengths
        L = int(lens.max()) if max_len is None and len(self) else int(max_len or 0)
        out = self.values.new_full((len(self), L, *self.values.shape[1:]), pad_value)
        mask = torch.arange(L, device=self.values.device)[None, :] < lens[:, None].to(self.values.device)
        out[mask] = self.values
        return out

    @staticmethod
    def cat(items: Sequence["Jagged"]) -> "Jagged":
        values = torch.cat([j.values for j in items], 0)
        offs = [items[0].offsets]
        base = items[0].offsets[-1]
        for j in items[1:]:
            offs.append(j.offsets[1:] + base)
            base = base + j.offsets[-1]
        return Jagged(values, torch.cat(offs))

    def __repr__(self):
        return f"Jagged(n={len(self)}, total={self.values.shape[0]}, dtype={self.values.dtype})"


TensorLike = Union[torch.Tensor, Jagged]


def _index_entry(v: TensorLike, idx) -> TensorLike:
    if isinstance(v, Jagged):
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(v))
            if step == 1:
                return v.slice(start, max(start, stop))
            idx = torch.arange(start, stop, step)
        return v.index(torch.as_tensor(idx))
    return v[idx]


class TensorBatch:
    """Minimal dict-of-tensors with a shared leading batch dimension (stand-in for ``tensordict.TensorDict``)."""

    def __init__(self, source: Optional[dict[str, TensorLike]] = None, batch_size: Optional[Sequence[int]] = None):
        self._d: dict[str, TensorLike] = dict(source or {})
        if batch_size is None:
            n = None
            for v in self._d.values():
                n = len(v) if isinstance(v, Jagged) else v.shape[0]
                break
            batch_size = (n if n is not None else 0,)
        if isinstance(batch_size, int):
            batch_size = (batch_size,)
        self.batch_size = torch.Size(batch_size)
        for k, v in self._d.items():
            n = len(v) if isinstance(v, Jagged) else v.shape[0]
            assert n == self.batch_size[0], f"entry {k} has batch {n}, expected {self.batch_size[0]}"

    # mapping interface
    def keys(self):
        return self._d.keys()

    def values(self):
        return self._d.values()

    def items(self):
        return self._d.items()

    def __contains__(self, k):
        return k in self._d

    def __iter__(self):
        return iter(self._d)

    def __len__(self):
        return self.batch_size[0]

    def __getitem__(self, k):
        if isinstance(k, str):
            return self._d[k]
        return TensorBatch({n: _index_entry(v, k) for n, v in self._d.items()}, batch_size=None if self._d else (0,))

    def __setitem__(self, k: str, v: TensorLike):
        n = len(v) if isinstance(v, Jagged) else v.shape[0]
        assert n == self.batch_size[0], f"entry {k} has batch {n}, expected {self.batch_size[0]}"
        self._d[k] = v

    def get(self, k, default=None):
        return self._d.get(k, default)

    def pop(self, k, *default):
        return self._d.pop(k, *default)

    def select(self, *keys) -> "TensorBatch":
        return TensorBatch({k: self._d[k] for k in keys}, batch_size=self.batch_size)

    def to(self, device) -> "TensorBatch":
        return TensorBatch({k: v.to(device) for k, v in self._d.items()}, batch_size=self.batch_size)

    def contiguous(self):
        return TensorBatch({k: (v if isinstance(v, Jagged) else v.contiguous()) for k, v in self._d.items()}, self.batch_size)

    @property
    def device(self):
        for v in self._d.values():
            return v.device
        return None

    def clone(self):
        return TensorBatch({k: (Jagged(v.values.clone(), v.offsets.clone()) if isinstance(v, Jagged) else v.clone()) for k, v in self._d.items()}, self.batch_size)

    def to_dict(self) -> dict:
        return dict(self._d)

    def __repr__(self):
        body = ", ".join(f"{k}: {tuple(v.shape) if isinstance(v, torch.Tensor) else v}" for k, v in self._d.items())
        return f"TensorBatch(batch_size={tuple(self.batch_size)}, {{{body}}})"

    @staticmethod
    def cat(items: Sequence["TensorBatch"]) -> "TensorBatch":
        keys = list(items[0].keys())
        out = {}
        for k in keys:
            vs = [it[k] for it in items]
            out[k] = Jagged.cat(vs) if isinstance(vs[0], Jagged) else torch.cat(vs, dim=0)
        return TensorBatch(out, batch_size=(sum(len(it) for it in items),))


# --------------------------------------------------------------------------------------------------------------
def union_tensor_dict(a: TensorBatch, b: TensorBatch) -> TensorBatch:
    """Merge ``b`` into ``a``; the same key must hold equal tensors in both."""
    assert a.batch_size == b.batch_size, f"batch sizes differ: {a.batch_size} vs {b.batch_size}"
    for k, v in b.items():
        if k in a:
            cur = a[k]
            same = (
                torch.equal(cur.values, v.values) and torch.equal(cur.offsets, v.offsets)
                if isinstance(cur, Jagged)
                else cur.shape == v.shape and torch.equal(cur, v)
            )
            assert same, f"key {k} present in both batches with different values"
        else:
            a[k] = v
    return a


def union_numpy_dict(a: dict[str, np.ndarray], b: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    for k, v in b.items():
        if k in a:
            assert isinstance(v, np.ndarray) and isinstance(a[k], np.ndarray)
            assert _np_equal(a[k], v), f"key {k} present in both non-tensor batches with different values"
        a[k] = v
    return a


def _np_equal(x: np.ndarray, y: np.ndarray) -> bool:
    if x.shape != y.shape:
        return False
    try:
        return bool(np.all(x == y))
    except Exception:
        return all(_py_equal(p, q) for p, q in zip(x.ravel(), y.ravel()))


def _py_equal(p, q) -> bool:
    try:
        r = p == q
        return bool(r.all()) if hasattr(r, "all") else bool(r)
    except Exception:
        return False


def _to_object_array(v, n: Optional[int] = None) -> np.ndarray:
    if isinstance(v, np.ndarray) and (v.dtype == object or n is None or v.shape[0] == n):
        return v
    arr = np.empty(len(v), dtype=object)
    for i, x in enumerate(v):
        arr[i] = x
    return arr


def collate_fn(samples: list[dict]) -> dict:
    """Stack tensor fields, turn everything else into object arrays (dataset → batch dictionary)."""
    tensors: dict[str, list] = {}
    others: dict[str, list] = {}
    for s in samples:
        for k, v in s.items():
            (tensors if isinstance(v, torch.Tensor) else others).setdefault(k, []).append(v)
    out: dict[str, Any] = {k: torch.stack(v, 0) for k, v in tensors.items()}
    for k, v in others.items():
        out[k] = _to_object_array(v)
    return out


# --------------------------------------------------------------------------------------------------------------
@dataclass
class DataProtoItem:
    batch: Optional[TensorBatch] = None
    non_tensor_batch: dict = field(default_factory=dict)
    meta_info: dict = field(default_factory=dict)


@dataclass
class DataProto:
    batch: Optional[TensorBatch] = None
    non_tensor_batch: dict = field(default_factory=dict)
    meta_info: dict = field(default_factory=dict)

    def __post_init__(self):
        self.check_consistency()

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(
        cls,
        tensors: Optional[dict[str, TensorLike]] = None,
        non_tensors: Optional[dict] = None,
        meta_info: Optional[dict] = None,
        num_batch_dims: int = 1,
        auto_padding: bool = False,
    ) -> "DataProto":
        tensors = tensors or {}
        non_tensors = non_tensors or {}
        assert num_batch_dims > 0
        if not tensors and not non_tensors:
            obj = cls(batch=None, non_tensor_batch={}, meta_info=dict(meta_info or {}))
        else:
            bs = None
            first = None
            for k, v in tensors.items():
                cur = (len(v),) if isinstance(v, Jagged) else tuple(v.shape[:num_batch_dims])
                if bs is None:
                    bs, first = cur, k
                assert cur == bs, f"tensor {k} has batch dims {cur}, but {first} has {bs}"
            nt = {k: _to_object_array(v) for k, v in non_tensors.items()}
            batch = TensorBatch(tensors, batch_size=bs) if tensors else None
            obj = cls(batch=batch, non_tensor_batch=nt, meta_info=dict(meta_info or {}))
        if auto_padding:
            obj.meta_info["_verl_auto_padding"] = True
        return obj

    @classmethod
    def from_single_dict(cls, data: dict, meta_info: Optional[dict] = None, auto_padding: bool = False) -> "DataProto":
        tensors, non_tensors = {}, {}
        for k, v in data.items():
            if isinstance(v, (torch.Tensor, Jagged)):
                tensors[k] = v
            elif isinstance(v, np.ndarray):
                non_tensors[k] = v
            else:
                raise ValueError(f"unsupported type {type(v)} for key {k}")
        return cls.from_dict(tensors, non_tensors, meta_info, auto_padding=auto_padding)

    @classmethod
    def from_tensordict(cls, td, meta_info: Optional[dict] = None) -> "DataProto":
        if isinstance(td, TensorBatch):
            return cls(batch=td, non_tensor_batch={}, meta_info=dict(meta_info or {}))
        return cls.from_single_dict(dict(td.items()), meta_info)

    def to_tensordict(self) -> TensorBatch:
        return self.batch

    # ------------------------------------------------------------------ basics
    def __len__(self) -> int:
        if self.batch is not None:
            return self.batch.batch_size[0]
        for v in self.non_tensor_batch.values():
            return v.shape[0]
        return 0

    def check_consistency(self):
        if self.batch is not None:
            assert len(self.batch.batch_size) >= 1
        n = len(self) if (self.batch is not None or self.non_tensor_batch) else None
        for k, v in self.non_tensor_batch.items():
            assert isinstance(v, np.ndarray), f"non-tensor entry {k} must be a numpy array, got {type(v)}"
            assert v.shape[0] == n, f"non-tensor entry {k} has length {v.shape[0]}, expected {n}"

    def __getitem__(self, item):
        if isinstance(item, slice):
            return self.slice(item.start, item.stop, item.step)
        if isinstance(item, (list, np.ndarray, torch.Tensor)):
            return self.select_idxs(item)
        if isinstance(item, (int, np.integer)):
            b = None
            if self.batch is not None:
                b = {k: (v.row(int(item)) if isinstance(v, Jagged) else v[int(item)]) for k, v in self.batch.items()}
            nt = {k: v[int(item)] for k, v in self.non_tensor_batch.items()}
            return DataProtoItem(batch=b, non_tensor_batch=nt, meta_info=self.meta_info)
        raise TypeError(f"indexing with {type(item)} is not supported")

    def slice(self, start=None, end=None, step=None) -> "DataProto":
        sl = slice(start, end, step)
        b = self.batch[sl] if self.batch is not None else None
        nt = {k: v[sl] for k, v in self.non_tensor_batch.items()}
        return type(self)(batch=b, non_tensor_batch=nt, meta_info=self.meta_info)

    def select_idxs(self, idxs) -> "DataProto":
        if isinstance(idxs, list):
            idxs = torch.tensor(idxs)
        if isinstance(idxs, np.ndarray):
            idxs = torch.from_numpy(idxs)
        idxs_np = idxs.detach().cpu().numpy()
        if idxs.dtype == torch.bool:
            idxs_t = torch.nonzero(idxs, as_tuple=False).flatten()
            idxs_np = idxs_t.cpu().numpy()
        else:
            idxs_t = idxs.to(torch.int64)
        b = None
        if self.batch is not None:
            dev = self.batch.device
            b = TensorBatch({k: _index_entry(v, idxs_t.to(dev) if not isinstance(v, Jagged) else idxs_t) for k, v in self.batch.items()},
                            batch_size=(len(idxs_np),))
        nt = {k: v[idxs_np] for k, v in self.non_tensor_batch.items()}
        return type(self)(batch=b, non_tensor_batch=nt, meta_info=self.meta_info)

    def to(self, device) -> "DataProto":
        if self.batch is not None:
            self.batch = self.batch.to(device)
        return self

    def select(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None, deepcopy=False) -> "DataProto":
        b = self.batch
        if batch_keys is not None and b is not None:
            b = b.select(*tuple(batch_keys))
        nt = self.non_tensor_batch
        if non_tensor_batch_keys is not None:
            nt = {k: v for k, v in nt.items() if k in non_tensor_batch_keys}
        mi = self.meta_info
        if meta_info_keys is not None:
            mi = {k: v for k, v in mi.items() if k in meta_info_keys}
        if deepcopy:
            nt, mi = copy.deepcopy(nt), copy.deepcopy(mi)
            b = b.clone() if b is not None else None
        return type(self)(batch=b, non_tensor_batch=dict(nt), meta_info=dict(mi))

    def pop(self, batch_keys=None, non_tensor_batch_keys=None, meta_info_keys=None) -> "DataProto":
        batch_keys = list(batch_keys or [])
        non_tensor_batch_keys = list(non_tensor_batch_keys or [])
        meta_info_keys = list(meta_info_keys or [])
        tensors = {k: self.batch.pop(k) for k in batch_keys}
        nt = {k: self.non_tensor_batch.pop(k) for k in non_tensor_batch_keys}
        mi = {k: self.meta_info.pop(k) for k in meta_info_keys}
        return DataProto.from_dict(tensors=tensors, non_tensors=nt, meta_info=mi)

    def rename(self, old_keys=None, new_keys=None) -> "DataProto":
        def as_list(x):
            if x is None:
                return []
            return [x] if isinstance(x, str) else list(x)

        old_keys, new_keys = as_list(old_keys), as_list(new_keys)
        assert len(old_keys) == len(new_keys)
        for o, n in zip(old_keys, new_keys):
            self.batch._d[n] = self.batch._d.pop(o)
        return self

    def union(self, other: "DataProto") -> "DataProto":
        if self.batch is None:
            self.batch = other.batch
        elif other.batch is not None:
            self.batch = union_tensor_dict(self.batch, other.batch)
        self.non_tensor_batch = union_numpy_dict(self.non_tensor_batch, other.non_tensor_batch)
        for k, v in other.meta_info.items():
            if k in self.meta_info and k != "metrics":
                assert _py_equal(self.meta_info[k], v), f"meta_info key {k} conflicts in union"
            self.meta_info[k] = v
        return self

    # ------------------------------------------------------------------ iteration
    def make_iterator(self, mini_batch_size: int, epochs: int, seed=None, dataloader_kwargs=None) -> Iterator["DataProto"]:
        n = len(self)
        assert n % mini_batch_size == 0, f"{n} % {mini_batch_size} != 0"
        dataloader_kwargs = dataloader_kwargs or {}
        shuffle = dataloader_kwargs.get("shuffle", True)
        gen = torch.Generator()
        if seed is not None:
            gen.manual_seed(int(seed))

        def it():
            for _ in range(epochs):
                order = torch.randperm(n, generator=gen) if shuffle else torch.arange(n)
                for s in range(0, n, mini_batch_size):
                    yield self.select_idxs(order[s : s + mini_batch_size])

        return iter(it())

    # ------------------------------------------------------------------ padding
    def is_padding_enabled(self) -> bool:
        return bool(self.meta_info.get("_verl_auto_padding", False)) or os.getenv("VERL_AUTO_PADDING", "").lower() in ("1", "true")

    def padding(self, padding_size: int, padding_candidate: str = "first"):
        if padding_size == 0:
            return
        src = self.select_idxs([0] if padding_candidate == "first" else [len(self) - 1])
        pad = src.repeat(padding_size)
        merged = DataProto.concat([self, pad])
        self.batch, self.non_tensor_batch = merged.batch, merged.non_tensor_batch

    # ------------------------------------------------------------------ split / merge
    def chunk(self, chunks: int) -> list["DataProto"]:
        n = len(self)
        if not self.is_padding_enabled():
            assert n % chunks == 0, f"only equal chunking is supported: len {n}, chunks {chunks}"
        size = math.ceil(n / chunks) if n else 0
        out = []
        for i in range(chunks):
            out.append(self.slice(i * size, min(n, (i + 1) * size)))
        return out

    def split(self, split_size: int) -> list["DataProto"]:
        return [self[i : i + split_size] for i in range(0, len(self), split_size)]

    @staticmethod
    def concat(data: list["DataProto"]) -> "DataProto":
        batches = [d.batch for d in data if d.batch is not None]
        b = TensorBatch.cat(batches) if batches else None
        nt: dict[str, np.ndarray] = {}
        keys = data[0].non_tensor_batch.keys() if data else []
        for k in keys:
            nt[k] = np.concatenate([d.non_tensor_batch[k] for d in data], axis=0)
        # meta_info: identical keys must agree, except "metrics" lists/dicts which are merged
        meta: dict[str, Any] = {}
        merged_metrics: list = []
        for d in data:
            for k, v in d.meta_info.items():
                if k == "metrics":
                    if isinstance(v, list):
                        merged_metrics.extend(v)
                    elif v is not None:
                        merged_metrics.append(v)
                    continue
                if k == "timing" and isinstance(v, dict):   # per-worker timings: keep every worker's value
                    t = meta.setdefault("timing", {})
                    for tk, tv in v.items():
                        t.setdefault(tk, [])
                        t[tk].extend(tv if isinstance(tv, list) else [tv])
                    continue
                if k in meta:
                    assert _py_equal(meta[k], v), f"meta_info key {k} differs between concatenated batches"
                else:
                    meta[k] = v
        if merged_metrics:
            if all(isinstance(m, dict) for m in merged_metrics):
                agg: dict[str, list] = {}
                for m in merged_metrics:
                    for mk, mv in m.items():
                        agg.setdefault(mk, [])
                        agg[mk].extend(mv if isinstance(mv, list) else [mv])
                meta["metrics"] = agg
            else:
                meta["metrics"] = merged_metrics
        cls = type(data[0]) if data else DataProto
        return cls(batch=b, non_tensor_batch=nt, meta_info=meta)

    def reorder(self, indices: torch.Tensor):
        idx_np = indices.detach().cpu().numpy()
        if self.batch is not None:
            self.batch = self.batch[indices]
        self.non_tensor_batch = {k: v[idx_np] for k, v in self.non_tensor_batch.items()}

    def repeat(self, repeat_times: int = 2, interleave: bool = True) -> "DataProto":
        n = len(self)
        idx = torch.arange(n).repeat_interleave(repeat_times) if interleave else torch.arange(n).repeat(repeat_times)
        out = self.select_idxs(idx)
        out.meta_info = self.meta_info
        return out

    def sample_level_repeat(self, repeat_times) -> "DataProto":
        rt = torch.as_tensor(repeat_times)
        idx = torch.arange(len(self)).repeat_interleave(rt)
        return self.select_idxs(idx)

    def unfold_column_chunks(self, n_split: int, split_keys=None) -> "DataProto":
        """Split dim 1 of the chosen keys into ``n_split`` parts and fold them into the batch dimension."""
        tensors = {}
        for k, v in self.batch.items():
            if split_keys is not None and k in split_keys:
                shape = list(v.shape)
                tensors[k] = v.reshape(shape[0] * n_split, shape[1] // n_split, *shape[2:])
            else:
                tensors[k] = v.repeat_interleave(n_split, dim=0)
        nt = {}
        for k, v in self.non_tensor_batch.items():
            if split_keys is not None and k in split_keys:
                nt[k] = v.reshape(v.shape[0] * n_split, v.shape[1] // n_split, *v.shape[2:])
            else:
                nt[k] = np.repeat(v, n_split, axis=0)
        return type(self)(batch=TensorBatch(tensors), non_tensor_batch=nt, meta_info=self.meta_info)

    def get_data_info(self) -> str:
        lines = ["batch"]
        if self.batch is not None:
            for k, v in self.batch.items():
                lines.append(f"  {k}: {tuple(v.shape) if isinstance(v, torch.Tensor) else v} ")
        lines.append("non_tensor_batch")
        for k, v in self.non_tensor_batch.items():
            lines.append(f"  {k}: ndarray{v.shape} ({v.dtype})")
        lines.append("meta_info")
        for k, v in self.meta_info.items():
            lines.append(f"  {k}: {type(v).__name__}")
        return "\n".join(lines)

    # ------------------------------------------------------------------ serialisation
    def __getstate__(self):
        method = os.getenv("VERL_DATAPROTO_SERIALIZATION_METHOD", "torch")
        tensors = None
        if self.batch is not None:
            plain = {}
            for k, v in self.batch.items():
                if isinstance(v, Jagged):
                    plain[k] = ("jagged", v.values.contiguous().cpu(), v.offsets.cpu())
                else:
                    plain[k] = ("dense", v.contiguous().cpu())
            if method == "numpy":
                def to_np(t):
                    return (t.view(torch.int16).numpy(), "bf16") if t.dtype == torch.bfloat16 else (t.numpy(), None)
                tensors = ("numpy", {k: (p[0], *[to_np(t) for t in p[1:]]) for k, p in plain.items()})
            else:
                buf = io.BytesIO()
                torch.save(plain, buf)
                tensors = ("torch", buf.getvalue())
        return tensors, self.non_tensor_batch, self.meta_info

    def __setstate__(self, state):
        tensors, nt, mi = state
        batch = None
        if tensors is not None:
            kind, payload = tensors
            if kind == "torch":
                plain = torch.load(io.BytesIO(payload), weights_only=False, map_location="cpu")
            else:
                def from_np(p):
                    arr, tag = p
                    t = torch.from_numpy(arr)
                    return t.view(torch.bfloat16) if tag == "bf16" else t
                plain = {k: (p[0], *[from_np(x) for x in p[1:]]) for k, p in payload.items()}
            d = {}
            for k, p in plain.items():
                d[k] = Jagged(p[1], p[2]) if p[0] == "jagged" else p[1]
            batch = TensorBatch(d) if d else None
        self.batch, self.non_tensor_batch, self.meta_info = batch, nt, mi

    def save_to_disk(self, filepath: str):
        with open(filepath, "wb") as f:
            pickle.dump(self, f)

    @staticmethod
    def load_from_disk(filepath: str) -> "DataProto":
        with open(filepath, "rb") as f:
            return pickle.load(f)

    def print_size(self, prefix: str = ""):
        t = sum(v.element_size() * v.numel() for v in self.batch.values() if isinstance(v, torch.Tensor)) if self.batch is not None else 0
        nt = sum(v.nbytes for v in self.non_tensor_batch.values())
        print(f"{prefix}tensor batch {t / 2**30:.3f} GiB, non-tensor batch {nt / 2**30:.3f} GiB")


# --------------------------------------------------------------------------------------------------------------
def pad_dataproto_to_divisor(data: DataProto, size_divisor: int) -> tuple[DataProto, int]:
    """Pad by cycling the batch from its start until ``len`` divides ``size_divisor``; returns (padded, pad_size)."""
    assert isinstance(data, DataProto)
    n = len(data)
    if n % size_divisor == 0:
        return data, 0
    pad = size_divisor - n % size_divisor
    parts, remaining = [], pad
    while remaining > 0:
        take = min(remaining, n)
        parts.append(data[:take])
        remaining -= take
    return DataProto.concat([data] + parts), pad


def unpad_dataproto(data: DataProto, pad_size: int) -> DataProto:
    return data[:-pad_size] if pad_size else data


# --------------------------------------------------------------------------------------------------------------
@dataclass
class DataProtoFuture:
    """Lazy handle on the outputs of several workers.

    ``futures`` is a list of objects exposing ``.result()`` (``concurrent.futures``-style) or plain values;
    ``collect_fn`` merges the list of worker outputs into one ``DataProto``; ``dispatch_fn`` optionally picks this
    consumer's chunk. ``get()`` materialises. Mirrors ``verl/protocol.py:1171`` with the worker-group's own futures
    in place of Ray object references.
    """

    collect_fn: Callable
    futures: list
    dispatch_fn: Optional[Callable] = None

    @staticmethod
    def concat(data: list) -> "DataProtoFuture":
        return DataProtoFuture(collect_fn=DataProto.concat, futures=data)

    def chunk(self, chunks: int) -> list["DataProtoFuture"]:
        from functools import partial

        def pick(x, i, chunks):
            return x.chunk(chunks=chunks)[i]

        return [DataProtoFuture(self.collect_fn, self.futures, partial(pick, i=i, chunks=chunks)) for i in range(chunks)]

    def get(self) -> DataProto:
        outs = [f.result() if hasattr(f, "result") else f for f in self.futures]
        for o in outs:
            assert isinstance(o, DataProto)
        out = self.collect_fn(outs)
        if self.dispatch_fn is not None:
            out = self.dispatch_fn(out)
        return out


def all_gather_data_proto(data: DataProto, process_group) -> None:
    """In-place all-gather of every entry across ``process_group`` (legacy SP data replication path)."""
    import torch.distributed as dist

    ws = dist.get_world_size(group=process_group)
    prev_dev = data.batch.device
    gathered = {}
    for k, v in data.batch.items():
        assert isinstance(v, torch.Tensor)
        bufs = [torch.empty_like(v) for _ in range(ws)]
        dist.all_gather(bufs, v.contiguous(), group=process_group)
        gathered[k] = torch.cat(bufs, 0)
    data.batch = TensorBatch(gathered).to(prev_dev)
    objs = [None] * ws
    dist.all_gather_object(objs, data.non_tensor_batch, group=process_group)
    data.non_tensor_batch = {k: np.concatenate([o[k] for o in objs]) for k in data.non_tensor_batch}
