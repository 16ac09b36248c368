"""Sparse weight synchronisation: after the first (dense) sync only the elements whose bit pattern changed are sent.

With a 1e-6 learning rate in bf16 most weights do not change bits between RL steps, so the delta is typically a few
per cent of the model. Sender side per tensor: one fused kernel compares against the snapshot of what the receivers
hold, compacts ``(int32 position, 16-bit value)`` pairs and refreshes the snapshot (``csrc/quant_sync.cu``; PyTorch
formulation on CPU). Receivers scatter the pairs into their copy. A per-tensor checksum of the sender's full tensor is
verified after applying; on mismatch or when the delta exceeds ``dense_threshold`` of the tensor, the tensor travels
dense. Reference: ``verl/checkpoint_engine/delta_sync/sparse_gather.py:41-137`` and ``delta_sharded`` backend.
"""

from __future__ import annotations

import time
from typing import Iterable, Iterator, Optional

import torch
import torch.distributed as dist

from verl_b200.ops import _ext

from .base import CheckpointEngine, CheckpointEngineRegistry

__all__ = ["DeltaShardedEngine", "delta_compact", "delta_apply", "tensor_checksum"]


def _as_i16(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().reshape(-1).view(torch.int16)


def tensor_checksum(t: torch.Tensor) -> int:
    """Order-independent 64-bit sum of the raw 16-bit words (cheap, catches any missed or misplaced element)."""
    return int(_as_i16(t).to(torch.int64).sum().item()) & 0xFFFFFFFFFFFFFFFF


def delta_compact(cur: torch.Tensor, snap: torch.Tensor, cap: Optional[int] = None):
    """Returns ``(count, positions int32 [k], values int16 [k])`` with ``k = min(count, cap)`` and refreshes ``snap``."""
    c, s = _as_i16(cur), _as_i16(snap)
    n = c.numel()
    cap = n if cap is None else min(cap, n)
    if c.is_cuda and _ext.available() and n % 8 == 0 and n < 2**31:
        pos = torch.empty(cap, dtype=torch.int32, device=c.device)
        val = torch.empty(cap, dtype=torch.int16, device=c.device)
        count = int(_ext.ops().delta_compact16(c, s, pos, val))
        k = min(count, cap)
        return count, pos[:k], val[:k]
    idx = torch.nonzero(c != s, as_tuple=False).reshape(-1)
    count = idx.numel()
    vals = c[idx]
    s.copy_(c)
    return count, idx[:cap].to(torch.int32), vals[:cap]


def delta_apply(dst: torch.Tensor, pos: torch.Tensor, val: torch.Tensor):
    d = dst.reshape(-1).view(torch.int16)
    if d.is_cuda and _ext.available() and pos.numel():
        _ext.ops().delta_apply16(d, pos.contiguous(), val.contiguous(), pos.numel())
    elif pos.numel():
        d[pos.long()] = val


@CheckpointEngineRegistry.register("delta_sharded")
class DeltaShardedEngine(CheckpointEngine):
    def __init__(self, group=None, src: int = 0, dense_threshold: float = 0.25, device: Optional[torch.device] = None, **kwargs):
        self.group, self.src, self.dense_threshold = group, src, dense_threshold
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and
                                 dist.get_backend(group) != "gloo" else torch.device("cpu"))
        self.snapshots: dict[str, torch.Tensor] = {}     # sender: what receivers hold; receiver: its own copy
        self.last_stats: dict = {}

    # ------------------------------------------------------------------ sender
    def send_weights(self, named_tensors: Iterable[tuple[str, torch.Tensor]]) -> dict:
        t0 = time.perf_counter()
        st = {"backend": "delta_sharded", "tensors": 0, "dense": 0, "changed": 0, "elements": 0, "bytes": 0}
        for name, t in named_tensors:
            t = t.detach()
            assert t.element_size() == 2, "delta sync works on 16-bit weights"
            st["tensors"] += 1
            st["elements"] += t.numel()
            snap = self.snapshots.get(name)
            mode, payload = "dense", None
            if snap is not None and snap.shape == t.shape:
                cap = max(8, int(t.numel() * self.dense_threshold))
                count, pos, val = delta_compact(t, snap, cap)
                if count <= cap:
                    mode, payload = "sparse", (pos, val)
                st["changed"] += count
            else:
                self.snapshots[name] = t.clone()
                st["changed"] += t.numel()
            hdr = {"name": name, "shape": tuple(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "mode": mode,
                   "count": 0 if payload is None else int(payload[0].numel()), "checksum": tensor_checksum(t), "last": False}
            dist.broadcast_object_list([hdr], src=self.src, group=self.group)
            if mode == "sparse":
                if hdr["count"]:
                    dist.broadcast(payload[0].to(self.device), src=self.src, group=self.group)
                    dist.broadcast(payload[1].to(self.device).contiguous().view(torch.uint8), src=self.src, group=self.group)
                st["bytes"] += hdr["count"] * 6
            else:
                st["dense"] += 1
                dist.broadcast(_as_i16(t).to(self.device).view(torch.uint8), src=self.src, group=self.group)
                st["bytes"] += t.numel() * 2
        dist.broadcast_object_list([{"last": True}], src=self.src, group=self.group)
        st["seconds"] = time.perf_counter() - t0
        st["changed_fraction"] = st["changed"] / max(1, st["elements"])
        self.last_stats = st
        return st

    # ------------------------------------------------------------------ receiver
    def receive_weights(self) -> Iterator[tuple[str, torch.Tensor]]:
        while True:
            box = [None]
            dist.broadcast_object_list(box, src=self.src, group=self.group)
            hdr = box[0]
            if hdr["last"]:
                return
            dt = getattr(torch, hdr["dtype"])
            name = hdr["name"]
            mine = self.snapshots.get(name)
            if hdr["mode"] == "sparse":
                if mine is None or tuple(mine.shape) != tuple(hdr["shape"]):
                    raise RuntimeError(f"delta for {name} arrived but this receiver holds no copy of it; run a dense sync first")
                if hdr["count"]:
                    pos = torch.empty(hdr["count"], dtype=torch.int32, device=self.device)
                    val = torch.empty(hdr["count"], dtype=torch.int16, device=self.device)
                    dist.broadcast(pos, src=self.src, group=self.group)
                    dist.broadcast(val.view(torch.uint8), src=self.src, group=self.group)
                    delta_apply(mine, pos.to(mine.device), val.to(mine.device))
            else:
                flat = torch.empty(int(torch.tensor(hdr["shape"]).prod()) if hdr["shape"] else 1, dtype=torch.int16, device=self.device)
                dist.broadcast(flat.view(torch.uint8), src=self.src, group=self.group)
                mine = flat.view(dt).reshape(hdr["shape"]).clone()
                self.snapshots[name] = mine
            if tensor_checksum(mine) != hdr["checksum"]:
                raise RuntimeError(f"checksum mismatch after applying the update of {name}")
            yield name, mine
