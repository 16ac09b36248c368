"""Geometry3K scoring: format (``<think>…</think>…\\boxed{}``) 10 % + accuracy 90 % (reference: ``utils/reward_score/geo3k.py``)."""

from __future__ import annotations

import re

from .math_reward import is_equiv, last_boxed_only_string, remove_boxed


def format_reward(s: str) -> float:
    return 1.0 if re.fullmatch(r"<think>.*</think>.*\\boxed\{.*\}.*", s, re.DOTALL) else 0.0


def acc_reward(s: str, gt: str) -> float:
    boxed = last_boxed_only_string(s)
    if boxed is None:
        return 0.0
    try:
        return 1.0 if is_equiv(remove_boxed(boxed), str(gt)) else 0.0
    except Exception:  # noqa: BLE001
        return 0.0


def compute_score(solution_str: str, ground_truth: str, format_weight: float = 0.1, **kwargs) -> float:
    return (1 - format_weight) * acc_reward(solution_str, ground_truth) + format_weight * format_reward(solution_str)
