"""Keep the activations saved for backward in pinned host memory instead of HBM.

``with offload_activations(...)`` wraps a forward region: every tensor autograd saves inside it (above a size
threshold, not a parameter) is copied to a pinned host buffer on a side stream and dropped from the device; backward
brings it back, prefetching the previously saved tensor (backward walks the saves in reverse order) so the copy of
layer i−1 overlaps the math of layer i. Reference: ``verl/utils/activation_offload.py:137-500`` (TE-style layer-group
double buffering for FSDP). On CPU tensors the context does nothing.
"""

from __future__ import annotations

import contextlib
from typing import Optional

import torch

__all__ = ["offload_activations", "ActivationOffloader", "enable_activation_offloading"]


class ActivationOffloader:
    def __init__(self, min_numel: int = 1 << 20, prefetch: bool = True):
        self.min_numel, self.prefetch = min_numel, prefetch
        self.stream: Optional[torch.cuda.Stream] = None
        self.saved: list = []           # [host tensor, device, event, device tensor or None]
        self.bytes_offloaded = 0

    def _ensure_stream(self):
        if self.stream is None:
            self.stream = torch.cuda.Stream()

    def pack(self, t: torch.Tensor):
        if (not t.is_cuda) or t.numel() < self.min_numel or isinstance(t, torch.nn.Parameter) or getattr(t, "_is_view_of_param", False) \
                or not t.is_contiguous():
            return t
        self._ensure_stream()
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            host.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        t.record_stream(self.stream)
        self.saved.append([host, t.device, ev, None])
        self.bytes_offloaded += t.numel() * t.element_size()
        return ("offloaded", len(self.saved) - 1)

    def _fetch(self, idx: int):
        ent = self.saved[idx]
        if ent[3] is None and ent[0] is not None:
            with torch.cuda.stream(self.stream):
                ent[2].wait(self.stream)
                ent[3] = ent[0].to(ent[1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
                ent[2] = ev

    def unpack(self, obj):
        if not (isinstance(obj, tuple) and len(obj) == 2 and obj[0] == "offloaded"):
            return obj
        idx = obj[1]
        self._fetch(idx)
        if self.prefetch and idx > 0:
            self._fetch(idx - 1)
        ent = self.saved[idx]
        ent[2].wait(torch.cuda.current_stream())
        out = ent[3]
        out.record_stream(torch.cuda.current_stream())
        ent[0], ent[3] = None, None      # host and device copies are released once consumed
        return out

    def reset(self):
        self.saved = []


@contextlib.contextmanager
def offload_activations(offloader: Optional[ActivationOffloader] = None, min_numel: int = 1 << 20):
    if not torch.cuda.is_available():
        yield None
        return
    off = offloader or ActivationOffloader(min_numel)
    with torch.autograd.graph.saved_tensors_hooks(off.pack, off.unpack):
        yield off


def enable_activation_offloading(model, min_numel: int = 1 << 20):
    """Wrap every decoder layer's forward in :func:`offload_activations` (one shared offloader per model)."""
    off = ActivationOffloader(min_numel)
    for layer in getattr(model, "layers", []):
        fwd = layer.forward

        def wrapped(*a, _f=fwd, **k):
            with offload_activations(off):
                return _f(*a, **k)

        layer.forward = wrapped
    model._activation_offloader = off
    return off
