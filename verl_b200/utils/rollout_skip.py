"""Dump the rollout output of the first steps to disk and replay it on later runs, skipping generation while the rest of
the pipeline is debugged (reference: ``verl/utils/skip/skip_manager.py``; config ``rollout.skip``)."""

from __future__ import annotations

import os
from typing import Callable

from verl_b200.protocol import DataProto

__all__ = ["SkipManager"]


class SkipManager:
    def __init__(self, enable: bool = False, dump_dir: str = "~/.verl_b200/rollout_dump", max_dump_step: int = 1, tag: str = "default"):
        self.enable, self.max_dump_step = bool(enable), int(max_dump_step)
        self.dir = os.path.join(os.path.expanduser(dump_dir), tag)
        self.hits = self.misses = 0

    @classmethod
    def from_config(cls, cfg, tag: str = "default") -> "SkipManager":
        get = cfg.get if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        return cls(get("enable", False), get("dump_dir", "~/.verl_b200/rollout_dump"), get("max_dump_step", 1), tag)

    def _path(self, step: int) -> str:
        return os.path.join(self.dir, f"gen_step_{step}.pt")

    def wrap(self, generate: Callable[[DataProto], DataProto]) -> Callable[[DataProto], DataProto]:
        if not self.enable:
            return generate

        def wrapped(prompts: DataProto) -> DataProto:
            step = int(prompts.meta_info.get("global_steps", 0))
            path = self._path(step)
            if os.path.exists(path):
                self.hits += 1
                out = DataProto.load_from_disk(path)
                if len(out) == len(prompts):
                    return out
            self.misses += 1
            out = generate(prompts)
            if step <= self.max_dump_step:
                os.makedirs(self.dir, exist_ok=True)
                out.save_to_disk(path)
            return out

        return wrapped
