"""Console logging that knows which rank is speaking.

`LocalLogger` and `concat_dict_to_str` are the console backend of `verl_b200.utils.tracking.Tracking`, re-exported under the module path
recipes import them from.  `RankGate` decides once whether a rank speaks; the print helpers and `DecoratorLoggerBase` (the base of
decorators such as the GPU-memory and timing loggers) are thin users of it.

Reference: ``verl/utils/logger/aggregate_logger.py:26-140`` (``LocalLogger``, ``DecoratorLoggerBase``, ``print_rank_0``,
``print_with_rank``, ``print_with_rank_and_timer``, ``log_with_rank``).
"""
from __future__ import annotations

import datetime
import logging
from typing import Optional

import torch.distributed as dist

from verl_b200.utils.tracking import LocalLogger, concat_dict_to_str  # noqa: F401  (re-exported)


def _current_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


class RankGate:
    """``speaks(rank)``: every rank, or only rank 0."""

    def __init__(self, only_rank_0: bool):
        self.only_rank_0 = bool(only_rank_0)

    def speaks(self, rank: int) -> bool:
        return (not self.only_rank_0) or int(rank) == 0


def print_rank_0(message) -> None:
    if _current_rank() == 0:
        print(message, flush=True)


def print_with_rank(message: str, rank: int = 0, log_only_rank_0: bool = False) -> None:
    if RankGate(log_only_rank_0).speaks(rank):
        print(f"[Rank {rank}] {message}", flush=True)


def print_with_rank_and_timer(message: str, rank: int = 0, log_only_rank_0: bool = False) -> None:
    if RankGate(log_only_rank_0).speaks(rank):
        now = datetime.datetime.now().strftime("%Y-%m-%d %H:%M:%S")
        print(f"[{now}] [Rank {rank}] {message}", flush=True)


def log_with_rank(message: str, rank: int, logger: logging.Logger, level: int = logging.INFO, log_only_rank_0: bool = False) -> None:
    if RankGate(log_only_rank_0).speaks(rank):
        logger.log(level, f"[Rank {rank}] {message}")


class DecoratorLoggerBase:
    """Base of decorators that report something about the call they wrap: ``self.logging_function(text)`` prints (no logger given) or logs
    at ``level``, prefixed with ``role``, on rank 0 only unless ``log_only_rank_0`` is off."""

    def __init__(self, role: str, logger: Optional[logging.Logger] = None, level: int = logging.DEBUG, rank: int = 0, log_only_rank_0: bool = True):
        self.role, self.logger, self.level, self.rank = role, logger, level, int(rank)
        self.log_only_rank_0 = log_only_rank_0
        self._gate = RankGate(log_only_rank_0)
        self.logging_function = self.log_by_print if logger is None else self.log_by_logging

    def log_by_print(self, log_str: str) -> None:
        if self._gate.speaks(self.rank):
            print(f"{self.role} {log_str}", flush=True)

    def log_by_logging(self, log_str: str) -> None:
        if self.logger is None:
            raise ValueError("this decorator was built without a logger")
        if self._gate.speaks(self.rank):
            self.logger.log(self.level, f"{self.role} {log_str}")
