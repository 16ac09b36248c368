"""An actor worker that keeps named host-memory copies of its weights.

``save_model_to_cpu(key)`` copies what this rank owns of the actor — the flat low-precision parameter buffer the model computes with and
this rank's fp32 master shard — into pinned host memory; ``restore_model_from_cpu(key)`` writes a copy back into the live buffers (the
parameters are views into the flat buffer, so nothing is re-bound) and ``clear_cpu_model(key)`` drops it.  A trainer that runs rollout
and training on separate devices uses it to try an update and roll it back, or to keep the weights of version ``n`` around while
version ``n+1`` trains.  The optimizer moments are left alone: a snapshot is a set of weights, not a training state (that is what a
checkpoint is for).

The copies are issued on the current stream and are complete when the call returns (one synchronise per call), so the next optimizer
step cannot race them.

Reference: ``verl/experimental/separation/engine_workers.py:36-169`` (``DetachActorWorker.save_model_to_cpu`` /
``restore_model_from_cpu`` / ``clear_cpu_model`` with per-strategy copy handlers); one handler suffices here because every engine keeps
its trainable weights in one flat buffer.
"""
from __future__ import annotations

import torch

from verl_b200.single_controller.base import Dispatch
from verl_b200.single_controller.base.decorator import register
from verl_b200.workers.engine_workers import ActorRolloutRefWorker


def _to_host(t: torch.Tensor) -> torch.Tensor:
    out = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)
    out.copy_(t, non_blocking=t.is_cuda)
    return out


class DetachActorWorker(ActorRolloutRefWorker):
    def _weights(self) -> dict[str, torch.Tensor]:
        if self.actor is None:
            raise RuntimeError("this worker holds no actor (role without 'actor', or init_model has not run)")
        eng = self.actor.engine
        store = getattr(eng, "store", None)
        if store is None or getattr(store, "flat", None) is None:
            raise NotImplementedError(f"{type(eng).__name__} does not keep its weights in a flat buffer; host snapshots are not available for it")
        live = {"flat": store.flat}
        if getattr(eng, "master", None) is not None:
            live["master"] = eng.master
        return live

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_model_to_cpu(self, n):
        if not hasattr(self, "cpu_saved_models"):
            self.cpu_saved_models = {}
        self.cpu_saved_models[n] = {k: _to_host(v) for k, v in self._weights().items()}
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
        return sum(v.numel() * v.element_size() for v in self.cpu_saved_models[n].values())

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def restore_model_from_cpu(self, n):
        saved = getattr(self, "cpu_saved_models", {}).get(n)
        if saved is None:
            return False
        live = self._weights()
        for k, v in saved.items():
            if live[k].shape != v.shape:
                raise RuntimeError(f"snapshot {n!r}: {k} has {tuple(v.shape)}, the engine now has {tuple(live[k].shape)}")
            live[k].copy_(v, non_blocking=live[k].is_cuda)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
        return True

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def clear_cpu_model(self, n):
        return getattr(self, "cpu_saved_models", {}).pop(n, None) is not None

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def saved_model_keys(self):
        return sorted(getattr(self, "cpu_saved_models", {}), key=str)
