"""The actor → rollout weight hand-off of one hybrid worker, behind one object the worker owns.

Which path runs depends on where the trainer keeps its weights and what the rollout replica holds
(``rollout.checkpoint_engine.backend``: ``naive`` = pick the in-process path below, ``nccl`` = always gather with
collectives, the baseline):

===============================  ==========================================================================================
trainer / rollout layout          path
===============================  ==========================================================================================
resident bf16 weights, TP = 1     nothing moves: the rollout engine reads the trainer's parameters (offloaded → brought back)
resident bf16 weights, TP > 1     ``refresh_rollout_shard``: one device copy of 1/tp of the layers
ZeRO-3 row shards (symmetric)     ``PeerReshardSync``: kernels read the peers' rows over NVLink straight into the rollout
                                  layout (full copy or TP slice) — no collective, no full-size intermediate
TP x PP trainer, LoRA, CPU ranks  per-tensor export (collective gather) streamed into the rollout copy, then re-cut for TP
===============================  ==========================================================================================

Reference: ``CheckpointEngineManager`` (``verl/checkpoint_engine/base.py:380-562``) and the naive colocated path of
``ActorRolloutRefWorker.update_weights`` (``verl/workers/engine_workers.py:734-836``), which always streams gathered
per-tensor parameters through CUDA-IPC buckets into the serving engine.
"""

from __future__ import annotations

import time
from typing import Optional

import torch
import torch.distributed as dist

__all__ = ["CheckpointEngineManager"]


class CheckpointEngineManager:
    def __init__(self, worker, backend: str = "naive"):
        self.worker = worker
        self.backend = str(backend or "naive")
        self.last_stats: dict = {}
        self._peer_sync = None

    # ------------------------------------------------------------------ replicas (API parity with the reference manager)
    def sleep_replicas(self):
        if self.worker.rollout is not None:
            self.worker.rollout.sleep()

    def wake_up_replicas(self):
        if self.worker.rollout is not None:
            self.worker.rollout.wake_up()

    # ------------------------------------------------------------------ hand-off
    def _uses_peer_reshard(self, eng) -> bool:
        return self.backend != "nccl" and bool(getattr(eng, "_zero3_rows", None)) and bool(getattr(eng, "_shard_dense", False))

    def update_weights(self) -> dict:
        w = self.worker
        t0 = time.perf_counter()
        stats = {"path": "none"}
        tp = getattr(w, "_rollout_tp", 1)
        if w.actor is not None and w.rollout is not None:
            eng = w.actor.engine
            cuda = torch.cuda.is_available()
            if getattr(w, "_rollout_owns_model", False):
                if self._uses_peer_reshard(eng):
                    from .reshard import PeerReshardSync

                    if self._peer_sync is None:
                        # with tensor-parallel replicas the kernels write this rank's slice directly; the replica's full copy
                        # only keeps the tensors the slice shares with it (embedding, final norm, output matrix)
                        self._peer_sync = PeerReshardSync(eng, w.rollout.model, w.rank % tp, tp)
                    stats = {"path": "peer_reshard", **self._peer_sync.sync()}
                    tp = 1                                  # the slice is already cut
                else:
                    target = getattr(w, "_rollout_sync_target", None) or getattr(w, "_rollout_full_model", None) or w.rollout.model
                    n = target.load_hf_stream(eng.get_per_tensor_param()[0])
                    stats = {"path": "per_tensor_gather", "tensors": n}
            elif not eng.store.flat.is_cuda and cuda:
                eng.to("cuda", model=True, optimizer=False, grad=False)
                w.rollout._graph = None
                stats = {"path": "resident_reload"}
            else:
                stats = {"path": "resident_shared"}
        if w.rollout is not None and tp > 1:
            from verl_b200.models.parallel_model import refresh_rollout_shard

            if not w._rollout_full_model.embed_tokens.is_cuda and torch.cuda.is_available():
                w.actor.engine.to("cuda", model=True, optimizer=False, grad=False)
            refresh_rollout_shard(w.rollout.model, w._rollout_full_model, w.rank % tp, tp)
            stats["tp_recut"] = True
        if dist.is_initialized():
            dist.barrier()
        stats["seconds_total"] = time.perf_counter() - t0
        self.last_stats = stats
        return stats
