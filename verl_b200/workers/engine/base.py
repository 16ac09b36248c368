"""Training-engine contract and registry.

An engine owns a model, its sharded optimizer state and its checkpoint logic and exposes a small, backend-agnostic
API to the role workers. Parity target: ``verl/workers/engine/base.py`` (BaseEngine :30-297, BaseEngineCtx :300-336,
EngineRegistry :339-445).
"""

from __future__ import annotations

import os
from abc import ABC, abstractmethod
from typing import Any, Callable, Generator, Optional

import torch

__all__ = ["BaseEngine", "BaseEngineCtx", "EngineRegistry"]


class BaseEngine(ABC):
    """Abstract training engine. Subclasses: ``fsdp`` (sharded data parallel), ``megatron`` (TP × PP × DP × EP)."""

    # ------------------------------------------------------------------ lifecycle
    @abstractmethod
    def initialize(self) -> None:
        """Build model, optimizer, LR schedule and checkpoint manager."""

    @property
    @abstractmethod
    def is_param_offload_enabled(self) -> bool: ...

    @property
    @abstractmethod
    def is_optimizer_offload_enabled(self) -> bool: ...

    def train_mode(self, **kwargs) -> "BaseEngineCtx":
        """Context manager: parameters, gradients and optimizer state resident on the device inside the block."""
        return BaseEngineCtx(self, mode="train", **kwargs)

    def eval_mode(self, **kwargs) -> "BaseEngineCtx":
        """Context manager: parameters resident on the device inside the block (no optimizer state)."""
        return BaseEngineCtx(self, mode="eval", **kwargs)

    # ------------------------------------------------------------------ compute
    @abstractmethod
    def forward_backward_batch(self, data, loss_function: Optional[Callable], forward_only: bool = False) -> dict:
        """Run all micro-batches of ``data``; returns ``{"model_output": {...}, "loss": [...], "metrics": {...}}``."""

    def train_batch(self, data, loss_function: Callable) -> dict:
        """One optimizer step on a mini-batch: zero_grad → forward/backward over micro-batches → step."""
        self.optimizer_zero_grad()
        out = self.forward_backward_batch(data, loss_function, forward_only=False)
        grad_norm = self.optimizer_step()
        if self.is_mp_src_rank_with_outputs():
            out.setdefault("metrics", {})["grad_norm"] = grad_norm
        return out

    def infer_batch(self, data, loss_function: Optional[Callable] = None) -> dict:
        with torch.no_grad():
            return self.forward_backward_batch(data, loss_function, forward_only=True)

    @abstractmethod
    def optimizer_zero_grad(self) -> None: ...

    @abstractmethod
    def optimizer_step(self) -> float:
        """Clip by global norm, skip on non-finite gradients, apply the update; returns the gradient norm."""

    @abstractmethod
    def lr_scheduler_step(self) -> float:
        """Advance the LR schedule; returns the new learning rate."""

    # ------------------------------------------------------------------ weights
    @abstractmethod
    def get_per_tensor_param(self, **kwargs) -> tuple[Generator[tuple[str, torch.Tensor], None, None], Optional[dict]]:
        """Generator of (HF tensor name, full tensor) for weight sync, plus an optional LoRA config."""

    def get_per_tensor_param_shard(self, **kwargs):
        raise NotImplementedError

    def get_per_tensor_param_delta_shard(self, **kwargs):
        raise NotImplementedError

    def disable_adapter(self):
        """Context manager that runs the base model without LoRA adapters (reference policy from the actor)."""
        from contextlib import nullcontext

        return nullcontext()

    # ------------------------------------------------------------------ placement
    @abstractmethod
    def to(self, device: str, model: bool = True, optimizer: bool = True, grad: bool = True) -> None: ...

    @abstractmethod
    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None, **kwargs) -> None: ...

    @abstractmethod
    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, del_local_after_load: bool = False,
                        **kwargs) -> None: ...

    # ------------------------------------------------------------------ topology
    @abstractmethod
    def get_data_parallel_rank(self) -> int: ...

    @abstractmethod
    def get_data_parallel_size(self) -> int: ...

    @abstractmethod
    def get_data_parallel_group(self): ...

    def is_mp_src_rank_with_outputs(self) -> bool:
        """True on the one rank of each model-parallel group whose outputs the controller collects."""
        return True


class BaseEngineCtx:
    """Moves state to the device on entry and back (if offloading is enabled) on exit."""

    def __init__(self, engine: BaseEngine, mode: str, **kwargs):
        assert mode in ("train", "eval")
        self.engine = engine
        self.mode = mode
        self.disable_auto_offload = kwargs.get("disable_auto_offload", False)

    def _device(self) -> str:
        from verl_b200.utils.device import get_device_name

        return get_device_name()

    def __enter__(self):
        e = self.engine
        e.mode = self.mode
        if not self.disable_auto_offload:
            if e.is_param_offload_enabled:
                e.to(self._device(), model=True, optimizer=False, grad=False)
            if self.mode == "train" and e.is_optimizer_offload_enabled:
                e.to(self._device(), model=False, optimizer=True, grad=True)
        return self

    def __exit__(self, exc_type, exc, tb):
        e = self.engine
        if not self.disable_auto_offload:
            if e.is_param_offload_enabled:
                e.to("cpu", model=True, optimizer=False, grad=False)
            if self.mode == "train" and e.is_optimizer_offload_enabled:
                e.to("cpu", model=False, optimizer=True, grad=True)
        e.mode = None
        return False


class EngineRegistry:
    """(model_type, backend, device) → engine class. ``VERL_ENGINE_DEVICE`` overrides device detection."""

    _engines: dict[tuple[str, str, str], type] = {}

    @classmethod
    def register(cls, model_type, backend, device="cuda"):
        model_types = [model_type] if isinstance(model_type, str) else list(model_type)
        backends = [backend] if isinstance(backend, str) else list(backend)
        devices = [device] if isinstance(device, str) else list(device)

        def deco(engine_cls):
            for m in model_types:
                for b in backends:
                    for d in devices:
                        cls._engines[(m, b, d)] = engine_cls
            return engine_cls

        return deco

    @classmethod
    def get_engine_cls(cls, model_type: str, backend: str):
        from verl_b200.utils.device import get_device_name

        device = os.environ.get("VERL_ENGINE_DEVICE", get_device_name())
        key = (model_type, backend, device)
        if key not in cls._engines:
            raise ValueError(f"no engine registered for {key}; known: {sorted(cls._engines)}")
        return cls._engines[key]

    @classmethod
    def new(cls, model_type: str, backend: str, *args, **kwargs) -> BaseEngine:
        # importing the implementations registers them
        import verl_b200.workers.engine.fsdp  # noqa: F401

        if backend == "megatron":
            import verl_b200.workers.engine.megatron  # noqa: F401
        elif not backend.startswith("fsdp"):
            import verl_b200.workers.engine.aliases  # noqa: F401 - third-party backend names of the reference

        engine_config = kwargs.get("engine_config", args[1] if len(args) > 1 else None)
        if backend == "megatron" and model_type == "language_model" and engine_config is not None:
            def mopt(key, default=1):
                v = engine_config.get(key, default) if hasattr(engine_config, "get") else getattr(engine_config, key, default)
                return int(v or default)

            ep = mopt("expert_model_parallel_size")
            if ep > 1:
                # expert parallelism over the data-parallel ranks with no tensor / pipeline / context split is exactly the layout of
                # the expert-parallel sharded engine (experts E/W per rank, dispatch + combine inside the grouped GEMMs): the
                # Megatron-style strategy names resolve to it. Expert parallelism inside a sub-group of the data-parallel ranks,
                # or combined with TP / PP / CP, is not built.
                import torch.distributed as dist

                world = dist.get_world_size() if dist.is_initialized() else int(os.environ.get("WORLD_SIZE", "1"))
                other = mopt("tensor_model_parallel_size") * mopt("pipeline_model_parallel_size") * mopt("context_parallel_size")
                if other != 1 or ep != world:
                    raise NotImplementedError(f"expert_model_parallel_size={ep} needs tensor = pipeline = context parallel size 1 and "
                                              f"expert_model_parallel_size == world size ({world}) in this build")
                import verl_b200.workers.engine.fsdp.zero3  # noqa: F401

                ec = dict(engine_config) if hasattr(engine_config, "keys") else {k: getattr(engine_config, k) for k in vars(engine_config)}
                ec["expert_parallel_size"] = ep
                if "engine_config" in kwargs:
                    kwargs["engine_config"] = ec
                else:
                    args = (args[0], ec) + tuple(args[2:])
                return cls.get_engine_cls(model_type, "fsdp_zero3")(*args, **kwargs)
        if backend in ("fsdp", "fsdp2") and model_type == "language_model" and engine_config is not None:
            def opt(key):
                return engine_config.get(key, False) if hasattr(engine_config, "get") else getattr(engine_config, key, False)

            if opt("zero3") or opt("reshard_after_forward") or int(opt("expert_parallel_size") or 1) > 1:     # ZeRO-3: row-sharded weights gathered inside the GEMMs
                import verl_b200.workers.engine.fsdp.zero3  # noqa: F401

                backend = "fsdp_zero3"
        return cls.get_engine_cls(model_type, backend)(*args, **kwargs)
