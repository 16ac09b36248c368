"""Precision debugger: per-module numeric fingerprints of selected training stages.

While a stage runs (``actor_update``, ``actor_compute_log_prob``, ``ref_compute_log_prob``, ``compute_values``,
``critic_update``), forward hooks on the model's leaf-level blocks record, for every output tensor, its shape, dtype, mean,
absolute maximum, L2 norm and the number of NaN / Inf entries; gradients of the parameters are fingerprinted the same way at
the end of a training stage. One JSON line per record goes to ``<save_path>/precision_rank<r>.jsonl``. Two runs (another
precision, another kernel build, another parallel layout) are compared by diffing the files — :func:`compare_dumps` reports
the first module whose fingerprint drifts beyond a tolerance.

The reference delegates this to the ``msprobe`` package (``verl/utils/profiler/precision_debugger_profile.py:68-230``,
stages at :40-60); here it is self-contained.
"""

from __future__ import annotations

import json
import os
from typing import Iterable, Optional

import torch

__all__ = ["PrecisionDebugger", "STAGES", "compare_dumps"]

STAGES = ("actor_update", "actor_compute_log_prob", "ref_compute_log_prob", "compute_values", "critic_update")


def _fingerprint(t: torch.Tensor) -> dict:
    x = t.detach().float()
    finite = torch.isfinite(x)
    xf = torch.where(finite, x, torch.zeros_like(x))
    return {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "mean": float(xf.mean()) if x.numel() else 0.0,
            "absmax": float(xf.abs().max()) if x.numel() else 0.0, "l2": float(xf.norm()), "nan": int(torch.isnan(x).sum()),
            "inf": int(torch.isinf(x).sum())}


class PrecisionDebugger:
    def __init__(self, rank: int, save_path: str, stages: Optional[Iterable[str]] = None, strict: bool = False, max_modules: int = 4096):
        unknown = set(stages or ()) - set(STAGES)
        if unknown:
            raise ValueError(f"Unknown precision_debugger stages: {sorted(unknown)}")
        self.rank, self.save_path = rank, save_path
        self.stages = set(stages) if stages else set(STAGES)
        self.strict, self.max_modules = strict, max_modules
        self._handles: list = []
        self._fp = None
        self._stage = None
        self._step = 0

    def should_run(self, stage: str) -> bool:
        if stage not in STAGES:
            if self.strict:
                raise ValueError(f"Unknown precision_debugger stage: {stage}")
            return False
        return stage in self.stages

    def _write(self, rec: dict):
        if self._fp is None:
            os.makedirs(self.save_path, exist_ok=True)
            self._fp = open(os.path.join(self.save_path, f"precision_rank{self.rank}.jsonl"), "a")
        self._fp.write(json.dumps(rec) + "\n")

    def start(self, stage: str, model: torch.nn.Module, step: int = 0):
        if not self.should_run(stage) or self._handles:
            return False
        self._stage, self._step = stage, step
        calls: dict = {}

        def hook(name):
            def fn(mod, inputs, output):
                outs = output if isinstance(output, (tuple, list)) else (output,)
                n = calls[name] = calls.get(name, 0) + 1
                for i, o in enumerate(outs):
                    if isinstance(o, torch.Tensor):
                        self._write({"step": self._step, "stage": self._stage, "kind": "forward", "module": name, "call": n, "output": i, **_fingerprint(o)})
            return fn

        for i, (name, mod) in enumerate(model.named_modules()):
            if i >= self.max_modules:
                break
            if name and not any(True for _ in mod.children()) or name.count(".") == 1:       # leaves and top-level blocks (layers.N)
                self._handles.append(mod.register_forward_hook(hook(name)))
        return True

    def stop(self, model: Optional[torch.nn.Module] = None):
        for h in self._handles:
            h.remove()
        self._handles = []
        if model is not None and self._stage in ("actor_update", "critic_update"):
            for name, p in model.named_parameters():
                g = getattr(p, "main_grad", None)
                g = g if g is not None else p.grad
                if g is not None:
                    self._write({"step": self._step, "stage": self._stage, "kind": "grad", "module": name, **_fingerprint(g)})
        if self._fp is not None:
            self._fp.flush()
        self._stage = None


def compare_dumps(path_a: str, path_b: str, rtol: float = 1e-2, atol: float = 1e-6) -> Optional[dict]:
    """First record (in file order) whose mean / absmax / l2 differ beyond ``atol + rtol·|a|`` or whose NaN / Inf counts
    differ; ``None`` when the dumps agree."""
    with open(path_a) as fa, open(path_b) as fb:
        for la, lb in zip(fa, fb):
            a, b = json.loads(la), json.loads(lb)
            if (a["module"], a["kind"]) != (b["module"], b["kind"]):
                return {"reason": "different module order", "a": a, "b": b}
            if a["nan"] != b["nan"] or a["inf"] != b["inf"]:
                return {"reason": "non-finite counts differ", "a": a, "b": b}
            for k in ("mean", "absmax", "l2"):
                if abs(a[k] - b[k]) > atol + rtol * abs(a[k]):
                    return {"reason": f"{k} differs", "a": a, "b": b}
    return None
