"""Split training primitives ("Tinker-style"): gradient clearing, forward/backward and the optimizer step as three separate
calls, so that a client can accumulate several forward/backward calls into one update and choose the step's optimizer
hyper-parameters at step time.

Parity target: ``verl/workers/engine_workers_tinker.py`` (``OptimStepParams`` :38-43, ``TinkerTrainingWorker`` :110-187,
``TinkerActorRolloutRefWorker`` :189-210). The engines here own their AdamW state directly (no ``torch.optim`` parameter
groups), so a step-time override is applied to the engine's hyper-parameter attributes for that one step.
"""

from __future__ import annotations

import time
from dataclasses import asdict, dataclass
from typing import Optional

import torch

from verl_b200.protocol import DataProto
from verl_b200.single_controller.base import Dispatch, register
from verl_b200.single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn
from verl_b200.workers.engine_workers import ActorRolloutRefWorker, TrainingWorker, _model_inputs, _to_host

__all__ = ["OptimStepParams", "TinkerTrainingWorker", "TinkerActorRolloutRefWorker"]


@dataclass
class OptimStepParams:
    """AdamW hyper-parameters of ONE optimizer step; ``None`` keeps the engine's configured value."""

    lr: Optional[float] = None
    eps: Optional[float] = None
    betas: Optional[tuple] = None
    weight_decay: Optional[float] = None

    def to_dict(self) -> dict:
        return asdict(self)


_ENGINE_ATTR = {"lr": ("lr",), "eps": ("adam_eps",), "weight_decay": ("weight_decay",), "betas": ("beta1", "beta2")}


def _apply_optim_step_params(engine, params) -> dict:
    """Override the engine's AdamW hyper-parameters; returns the previous values so that the caller can restore them."""
    if params is None:
        return {}
    if hasattr(params, "to_dict"):
        params = params.to_dict()
    if not isinstance(params, dict):
        raise TypeError(f"optim_step_params must be a dict, got {type(params)}")
    saved = {}
    for key, value in params.items():
        if value is None:
            continue
        if key not in _ENGINE_ATTR:
            raise ValueError(f"unsupported optim_step_params key: {key!r} (known: {sorted(_ENGINE_ATTR)})")
        attrs = _ENGINE_ATTR[key]
        if key == "betas":
            if not (isinstance(value, (tuple, list)) and len(value) == 2):
                raise TypeError("optim_step_params['betas'] must be a pair of floats")
            vals = [float(value[0]), float(value[1])]
        else:
            if not isinstance(value, (int, float)) or isinstance(value, bool):
                raise TypeError(f"optim_step_params type mismatch for {key!r}: got {type(value).__name__}, expected float")
            vals = [float(value)]
        for a, v in zip(attrs, vals):
            saved[a] = getattr(engine, a)
            setattr(engine, a, v)
    return saved


class TinkerTrainingWorker(TrainingWorker):
    """:class:`TrainingWorker` plus ``optimizer_zero_grad`` / ``forward_backward`` / ``optimizer_step``."""

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_zero_grad(self) -> None:
        with self.engine.train_mode():
            self.engine.optimizer_zero_grad()

    def forward_backward(self, data: DataProto) -> DataProto:
        """Forward + backward over the micro-batches of ``data``; gradients add to what is already accumulated. Returns the
        per-token model outputs (log-probs, entropy when asked for) and the loss metrics — the client sees them after backward."""
        assert self.loss_fn is not None, "loss function can't be None when calling forward_backward"
        assert not getattr(self.engine, "forward_only", False), "can't run forward_backward on a forward-only engine"
        meta = self._batch_meta(data, "ppo_")
        d = DataProto(batch=data.batch, non_tensor_batch=_model_inputs(data), meta_info=meta)
        t0 = time.perf_counter()
        with self.engine.train_mode():
            out = self.engine.forward_backward_batch(d, self.loss_fn, forward_only=False)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if not self.engine.is_mp_src_rank_with_outputs():
            return DataProto(batch=None, non_tensor_batch={}, meta_info={"metrics": {}})
        tensors = {k: _to_host(v) for k, v in out["model_output"].items() if isinstance(v, torch.Tensor) and v.shape[:1] == (len(data),)}
        n_tok = int(data.batch["attention_mask"].sum())
        metrics = self._postprocess_metrics(dict(out["metrics"]), n_tok, dt, forward_only=False)
        metrics["loss"] = float(sum(out["loss"]))
        return DataProto.from_dict(tensors=tensors, meta_info={"metrics": metrics})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_step(self, optim_step_params=None) -> dict:
        """One optimizer step on the accumulated gradients, optionally with this step's own lr / eps / betas / weight decay."""
        eng = self.engine
        with eng.train_mode():
            saved = _apply_optim_step_params(eng, optim_step_params)
            try:
                if optim_step_params is not None and (optim_step_params.get("lr") if isinstance(optim_step_params, dict) else optim_step_params.lr) is not None:
                    # the override replaces the schedule's value for this step
                    lr_of = eng.current_lr
                    eng.current_lr = lambda: eng.lr
                    try:
                        grad_norm = eng.optimizer_step()
                    finally:
                        eng.current_lr = lr_of
                else:
                    grad_norm = eng.optimizer_step()
            finally:
                for a, v in saved.items():
                    setattr(eng, a, v)
        return {"grad_norm": grad_norm} if grad_norm is not None and eng.is_mp_src_rank_with_outputs() else {}


class TinkerActorRolloutRefWorker(ActorRolloutRefWorker):
    """Hybrid worker whose actor exposes the split primitives (``actor_worker_cls`` = :class:`TinkerTrainingWorker`)."""

    actor_worker_cls = TinkerTrainingWorker

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_zero_grad(self) -> None:
        assert "actor" in self.role, "optimizer_zero_grad only supports the actor role"
        return self.actor.optimizer_zero_grad()

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("actor"))
    def forward_backward(self, data: DataProto) -> DataProto:
        assert "actor" in self.role, "forward_backward only supports the actor role"
        meta = dict(data.meta_info)
        meta.setdefault("temperature", float(self.config.get("rollout", {}).get("temperature", 1.0)) if hasattr(self.config, "get") else 1.0)
        replay = self._router_replay_mode() in ("R2", "R3")
        d = DataProto(batch=data.batch if replay else self._without_routing(data.batch), non_tensor_batch=data.non_tensor_batch, meta_info=meta)
        return self.actor.forward_backward(d)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def optimizer_step(self, optim_step_params=None) -> dict:
        assert "actor" in self.role, "optimizer_step only supports the actor role"
        return self.actor.optimizer_step(optim_step_params=optim_step_params)
