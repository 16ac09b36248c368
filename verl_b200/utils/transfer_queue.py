"""In-process TransferQueue: a partitioned key→fields store with per-key tags, the data plane of the v1 trainers.

The reference talks to an external TransferQueue service (``verl/utils/transferqueue_utils.py:160-347``: ``tqbridge``
turns worker methods that receive ``KVBatchMeta`` into fetch → run → write-back). Here the store lives in the
controller process (each SPMD rank keeps its own, fed identically), which is all the single-box layouts need; the
interface (``kv_put / kv_get / kv_tags / kv_clear``, ``KVBatchMeta``, ``tqbridge``) is what a remote implementation
would have to provide.
"""

from __future__ import annotations

import functools
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Optional

import numpy as np
import torch

from verl_b200.protocol import DataProto

__all__ = ["TransferQueue", "KVBatchMeta", "get_transfer_queue", "tqbridge"]


@dataclass
class KVBatchMeta:
    """Names a batch without carrying it: a partition, the sample keys (row order) and the fields of interest."""

    partition_id: str
    keys: list
    fields: Optional[list] = None
    extra_info: dict = field(default_factory=dict)

    def __len__(self):
        return len(self.keys)

    def select(self, fields: Iterable[str]) -> "KVBatchMeta":
        return KVBatchMeta(self.partition_id, list(self.keys), list(fields), dict(self.extra_info))


class TransferQueue:
    def __init__(self):
        self._lock = threading.Condition()
        self._data: dict[str, dict[str, dict[str, Any]]] = {}
        self._tags: dict[str, dict[str, dict[str, Any]]] = {}

    # ------------------------------------------------------------------ writes
    def kv_put(self, partition_id: str, key: str, fields: Optional[dict] = None, tags: Optional[dict] = None):
        with self._lock:
            self._data.setdefault(partition_id, {}).setdefault(key, {}).update(fields or {})
            self._tags.setdefault(partition_id, {}).setdefault(key, {}).update(tags or {})
            self._lock.notify_all()

    def kv_batch_put(self, meta: KVBatchMeta, data: DataProto, tags: Optional[dict] = None):
        """Row i of ``data`` is written under ``meta.keys[i]`` (tensor fields per row, non-tensor fields as objects)."""
        assert len(data) == len(meta.keys)
        for i, k in enumerate(meta.keys):
            row = {name: t[i].clone() for name, t in (data.batch.items() if data.batch is not None else [])}
            row.update({name: v[i] for name, v in data.non_tensor_batch.items()})
            self.kv_put(meta.partition_id, k, row, tags)

    def kv_clear(self, partition_id: str, keys: Optional[Iterable[str]] = None):
        with self._lock:
            if keys is None:
                self._data.pop(partition_id, None)
                self._tags.pop(partition_id, None)
            else:
                for k in keys:
                    self._data.get(partition_id, {}).pop(k, None)
                    self._tags.get(partition_id, {}).pop(k, None)

    # ------------------------------------------------------------------ reads
    def kv_tags(self, partition_id: str) -> dict[str, dict]:
        with self._lock:
            return {k: dict(v) for k, v in self._tags.get(partition_id, {}).items()}

    def kv_get(self, meta: KVBatchMeta) -> DataProto:
        with self._lock:
            rows = [self._data[meta.partition_id][k] for k in meta.keys]
        names = meta.fields if meta.fields is not None else sorted(set().union(*[r.keys() for r in rows])) if rows else []
        tensors, non_tensors = {}, {}
        for name in names:
            vals = [r[name] for r in rows]
            if all(isinstance(v, torch.Tensor) for v in vals):
                tensors[name] = torch.stack(vals)
            else:
                arr = np.empty(len(vals), dtype=object)
                for i, v in enumerate(vals):
                    arr[i] = v
                non_tensors[name] = arr
        return DataProto.from_dict(tensors=tensors or None, non_tensors=non_tensors, meta_info=dict(meta.extra_info))

    def wait(self, predicate: Callable[[], bool], timeout: Optional[float] = None) -> bool:
        with self._lock:
            return self._lock.wait_for(predicate, timeout)

    def size(self, partition_id: str) -> int:
        with self._lock:
            return len(self._data.get(partition_id, {}))


_TQ: Optional[TransferQueue] = None


def get_transfer_queue() -> TransferQueue:
    global _TQ
    if _TQ is None:
        _TQ = TransferQueue()
    return _TQ


def tqbridge(put_data: bool = True):
    """Decorator for ``fn(self, data: DataProto, ...) -> DataProto``: when called with a ``KVBatchMeta`` instead, fetch the
    named fields from the queue, run, write the returned tensor fields back under the same keys and return the meta
    (extended with the new field names). Plain ``DataProto`` calls pass through untouched."""

    def deco(fn):
        @functools.wraps(fn)
        def wrapper(self, data, *args, **kwargs):
            if not isinstance(data, KVBatchMeta):
                return fn(self, data, *args, **kwargs)
            tq = get_transfer_queue()
            out = fn(self, tq.kv_get(data), *args, **kwargs)
            new_fields = []
            if put_data and isinstance(out, DataProto) and out.batch is not None and len(out) == len(data.keys):
                tq.kv_batch_put(data, out)
                new_fields = list(out.batch.keys()) + list(out.non_tensor_batch.keys())
            meta = KVBatchMeta(data.partition_id, list(data.keys), (list(data.fields or []) + new_fields) or None, dict(data.extra_info))
            if isinstance(out, DataProto):
                meta.extra_info.update(out.meta_info or {})
            return meta

        return wrapper

    return deco
