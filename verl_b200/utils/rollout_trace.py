"""Per-request rollout traces (reference: ``verl/utils/rollout_trace.py:31-364``: weave / mlflow / trackio backends and
the ``rollout_trace_op`` decorator). The built-in backend writes JSON lines; ``weave`` and ``mlflow`` are used when those
packages are importable. ``TrajectoryTracker`` keeps tensors of named pipeline points for offline diffing."""

from __future__ import annotations

import contextlib
import contextvars
import functools
import inspect
import json
import os
import time
from typing import Optional

import torch

__all__ = ["RolloutTraceConfig", "rollout_trace_attr", "rollout_trace_op", "TrajectoryTracker"]

_attrs: contextvars.ContextVar = contextvars.ContextVar("rollout_trace_attrs", default={})


class RolloutTraceConfig:
    """Process-wide singleton: ``RolloutTraceConfig.init(project, experiment, backend, token2text, path)``."""

    backend: Optional[str] = None
    token2text: bool = False
    project = experiment = None
    path: Optional[str] = None
    _fh = None

    @classmethod
    def init(cls, project: str, experiment: str, backend: Optional[str], token2text: bool = False, path: Optional[str] = None):
        cls.project, cls.experiment, cls.backend, cls.token2text = project, experiment, backend, token2text
        if backend in ("jsonl", "file"):
            cls.path = path or os.path.join(os.path.expanduser("~/.verl_b200/traces"), project, f"{experiment}.jsonl")
            os.makedirs(os.path.dirname(cls.path), exist_ok=True)
            cls._fh = open(cls.path, "a")
        elif backend == "weave":
            import weave

            weave.init(project)
        elif backend == "mlflow":
            import mlflow

            mlflow.set_experiment(project)
        elif backend is not None:
            raise ValueError(f"unknown trace backend {backend!r}")

    @classmethod
    def reset(cls):
        if cls._fh:
            cls._fh.close()
        cls.backend, cls._fh, cls.path = None, None, None

    @classmethod
    def emit(cls, record: dict):
        if cls._fh is not None:
            cls._fh.write(json.dumps(record, default=str) + "\n")
            cls._fh.flush()


@contextlib.contextmanager
def rollout_trace_attr(sample_index=None, step=None, rollout_n=None, name: str = "rollout_trace", validate: bool = False):
    """Attach sample coordinates to every traced call made inside the block."""
    tok = _attrs.set({"sample_index": sample_index, "step": step, "rollout_n": rollout_n, "name": name, "validate": validate})
    try:
        yield
    finally:
        _attrs.reset(tok)


def _plain(x):
    if isinstance(x, torch.Tensor):
        return x.tolist() if x.numel() <= 4096 else f"<tensor {tuple(x.shape)}>"
    if hasattr(x, "__dict__") and not isinstance(x, type):
        return {k: _plain(v) for k, v in vars(x).items() if not k.startswith("_")}
    if isinstance(x, (list, tuple)):
        return [_plain(v) for v in x]
    if isinstance(x, dict):
        return {k: _plain(v) for k, v in x.items()}
    return x


def rollout_trace_op(fn):
    """Decorator for (async) methods of agent loops / servers: records inputs, output and latency per call."""

    def record(self, args, kwargs, out, t0, err=None):
        if RolloutTraceConfig.backend is None:
            return
        names = list(inspect.signature(fn).parameters)[1:]
        inputs = {n: _plain(a) for n, a in zip(names, args)}
        inputs.update({k: _plain(v) for k, v in kwargs.items()})
        rec = {"op": fn.__qualname__, "attrs": dict(_attrs.get()), "inputs": inputs, "output": _plain(out), "seconds": time.time() - t0}
        if err is not None:
            rec["error"] = repr(err)
        tok = getattr(self, "tokenizer", None)
        if RolloutTraceConfig.token2text and tok is not None and hasattr(out, "token_ids"):
            rec["output_text"] = tok.decode(out.token_ids)
        RolloutTraceConfig.emit(rec)

    if inspect.iscoroutinefunction(fn):
        @functools.wraps(fn)
        async def aw(self, *args, **kwargs):
            t0 = time.time()
            try:
                out = await fn(self, *args, **kwargs)
            except Exception as e:
                record(self, args, kwargs, None, t0, e)
                raise
            record(self, args, kwargs, out, t0)
            return out

        return aw

    @functools.wraps(fn)
    def w(self, *args, **kwargs):
        t0 = time.time()
        try:
            out = fn(self, *args, **kwargs)
        except Exception as e:
            record(self, args, kwargs, None, t0, e)
            raise
        record(self, args, kwargs, out, t0)
        return out

    return w


class TrajectoryTracker:
    """Keeps CPU copies of tensors at named points of a step and writes them as one file per step (numerics bisecting)."""

    def __init__(self, dump_dir: Optional[str] = None, enable: bool = True):
        self.dump_dir, self.enable = dump_dir, enable
        self.store: dict[str, torch.Tensor] = {}

    def track(self, name: str, value):
        if self.enable:
            self.store[name] = value.detach().to("cpu", copy=True) if isinstance(value, torch.Tensor) else value

    def dump(self, step: int) -> Optional[str]:
        if not self.enable or self.dump_dir is None:
            return None
        os.makedirs(self.dump_dir, exist_ok=True)
        path = os.path.join(self.dump_dir, f"trajectory_step_{step}.pt")
        torch.save(self.store, path)
        self.store = {}
        return path

    @staticmethod
    def compare(a: dict, b: dict, rtol: float = 1e-5, atol: float = 1e-6) -> dict:
        out = {}
        for k in sorted(set(a) & set(b)):
            if isinstance(a[k], torch.Tensor) and isinstance(b[k], torch.Tensor) and a[k].shape == b[k].shape:
                d = (a[k].float() - b[k].float()).abs()
                out[k] = {"max_abs": float(d.max()) if d.numel() else 0.0, "close": bool(torch.allclose(a[k].float(), b[k].float(), rtol=rtol, atol=atol))}
        return out
