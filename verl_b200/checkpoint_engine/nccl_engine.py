"""Dense bucketed broadcast of the weights over a torch.distributed process group (reference:
``verl/checkpoint_engine/nccl_checkpoint_engine.py:106-429`` — uint8 buckets of ``update_weights_bucket_megabytes``,
double buffering, metadata over a side channel; here the side channel is an object broadcast on the same group)."""

from __future__ import annotations

import time
from typing import Iterable, Iterator, Optional

import torch
import torch.distributed as dist

from .base import CheckpointEngine, CheckpointEngineRegistry

__all__ = ["BucketedBroadcastEngine"]

_ALIGN = 256


def _pad(n: int) -> int:
    return -(-n // _ALIGN) * _ALIGN


@CheckpointEngineRegistry.register("nccl")
class BucketedBroadcastEngine(CheckpointEngine):
    def __init__(self, group=None, src: int = 0, bucket_megabytes: int = 2048, device: Optional[torch.device] = None, **kwargs):
        self.group, self.src = group, src
        self.bucket_bytes = int(bucket_megabytes) * (1 << 20)
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and
                                 dist.get_backend(group) != "gloo" else torch.device("cpu"))
        self._buckets = [None, None]

    def _bucket(self, i: int, nbytes: int) -> torch.Tensor:
        b = self._buckets[i]
        if b is None or b.numel() < nbytes:
            b = torch.empty(max(nbytes, min(self.bucket_bytes, 1 << 26)), dtype=torch.uint8, device=self.device)
            self._buckets[i] = b
        return b

    # ------------------------------------------------------------------ sender
    def send_weights(self, named_tensors: Iterable[tuple[str, torch.Tensor]]) -> dict:
        t0 = time.perf_counter()
        stats = {"backend": "nccl", "buckets": 0, "bytes": 0, "tensors": 0}
        meta, off, which = [], 0, 0
        buf = self._bucket(which, self.bucket_bytes if self.bucket_bytes < (1 << 26) else 1 << 26)
        pending = None

        def flush(last: bool):
            nonlocal meta, off, which, buf, pending
            if pending is not None:
                pending.wait()
            dist.broadcast_object_list([{"meta": meta, "nbytes": off, "last": last}], src=self.src, group=self.group)
            if off:
                pending = dist.broadcast(buf[:off], src=self.src, group=self.group, async_op=True)
            stats["buckets"] += 1
            stats["bytes"] += off
            meta, off = [], 0
            which ^= 1
            buf = self._bucket(which, buf.numel())

        for name, t in named_tensors:
            t = t.detach()
            nbytes = t.numel() * t.element_size()
            if off and off + _pad(nbytes) > buf.numel():
                flush(False)
            if _pad(nbytes) > buf.numel():
                buf = self._bucket(which, _pad(nbytes))
            buf[off : off + nbytes].copy_(t.contiguous().reshape(-1).view(torch.uint8), non_blocking=True)
            meta.append((name, tuple(t.shape), str(t.dtype).replace("torch.", ""), off, nbytes))
            off += _pad(nbytes)
            stats["tensors"] += 1
        flush(True)
        if pending is not None:
            pending.wait()
        stats["seconds"] = time.perf_counter() - t0
        return stats

    # ------------------------------------------------------------------ receiver
    def receive_weights(self) -> Iterator[tuple[str, torch.Tensor]]:
        which = 0
        while True:
            box = [None]
            dist.broadcast_object_list(box, src=self.src, group=self.group)
            hdr = box[0]
            if hdr["nbytes"]:
                buf = self._bucket(which, hdr["nbytes"])
                dist.broadcast(buf[: hdr["nbytes"]], src=self.src, group=self.group)
                for name, shape, dt, off, nbytes in hdr["meta"]:
                    yield name, buf[off : off + nbytes].view(getattr(torch, dt)).reshape(shape)
                which ^= 1
            if hdr["last"]:
                return
