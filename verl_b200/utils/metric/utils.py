"""Metric values that remember how they must be aggregated across micro-batches and data-parallel ranks.

Parity target: ``verl/utils/metric/utils.py`` (reduce_metrics :25, AggregationType :61, Metric :72).
"""

from __future__ import annotations

from enum import Enum
from typing import Any, Iterable, Union

import numpy as np
import torch

__all__ = ["AggregationType", "Metric", "reduce_metrics"]


class AggregationType(str, Enum):
    MEAN = "mean"
    SUM = "sum"
    MIN = "min"
    MAX = "max"


class Metric:
    """A list of scalar observations plus the reduction that turns them into one number."""

    def __init__(self, aggregation: Union[str, AggregationType], value=None):
        self.aggregation = AggregationType(aggregation)
        self.values: list[float] = []
        if value is not None:
            self.append(value)

    def append(self, value):
        if isinstance(value, Metric):
            self.extend(value)
        elif isinstance(value, (list, tuple)):
            for v in value:
                self.append(v)
        else:
            self.values.append(float(value.detach().item()) if torch.is_tensor(value) else float(value))

    def extend(self, other: "Metric"):
        assert other.aggregation == self.aggregation, "cannot merge metrics with different aggregation"
        self.values.extend(other.values)

    def aggregate(self) -> float:
        if not self.values:
            return float("nan")
        a = np.asarray(self.values, dtype=np.float64)
        return float({"mean": a.mean, "sum": a.sum, "min": a.min, "max": a.max}[self.aggregation.value]())

    @classmethod
    def aggregate_dp(cls, per_rank: Iterable["Metric"]) -> "Metric":
        per_rank = list(per_rank)
        out = cls(per_rank[0].aggregation)
        for m in per_rank:
            out.extend(m)
        return out

    def __repr__(self):
        return f"Metric({self.aggregation.value}, n={len(self.values)})"


def reduce_metrics(metrics: dict[str, Any]) -> dict[str, float]:
    """Lists → mean (``*_max`` / ``*_min`` suffixed keys → max / min); ``Metric`` → its own aggregation."""
    out = {}
    for k, v in metrics.items():
        if isinstance(v, Metric):
            out[k] = v.aggregate()
        elif isinstance(v, (list, tuple, np.ndarray)):
            if len(v) == 0:
                out[k] = float("nan")
            elif k.endswith("/max") or k.endswith("_max"):
                out[k] = float(np.max(v))
            elif k.endswith("/min") or k.endswith("_min"):
                out[k] = float(np.min(v))
            else:
                out[k] = float(np.mean(v))
        else:
            out[k] = float(v.item()) if torch.is_tensor(v) else v
    return out
