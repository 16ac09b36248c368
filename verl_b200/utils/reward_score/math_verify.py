"""Symbolic answer check through the ``math-verify`` package: the boxed ground truth and the model output are parsed to
expressions (LaTeX and plain) and compared for mathematical equivalence. Parsing runs in a small pool of spawned worker
processes because the package's own time-outs need ``signal.alarm``, which only works on a process's main thread; a hung
comparison costs ``timeout`` seconds and scores ``timeout_score``. Reference: ``verl/utils/reward_score/math_verify.py``.

The package is optional: without it :func:`available` is False and :func:`compute_score` raises ``ImportError`` so that a
mis-configured run fails at the first sample instead of silently scoring zeros.
"""

from __future__ import annotations

import multiprocessing
import threading
from concurrent.futures import ProcessPoolExecutor
from concurrent.futures import TimeoutError as FuturesTimeout

__all__ = ["compute_score", "available"]

_pool = None
_lock = threading.Lock()


def available() -> bool:
    try:
        import math_verify  # noqa: F401

        return True
    except ImportError:
        return False


def _workers():
    global _pool
    with _lock:
        if _pool is None:
            _pool = ProcessPoolExecutor(max_workers=4, mp_context=multiprocessing.get_context("spawn"))
    return _pool


def _verify(gold_boxed: str, output: str) -> float:
    from math_verify.grader import verify
    from math_verify.parser import ExprExtractionConfig, LatexExtractionConfig, parse

    gold = parse(gold_boxed, (LatexExtractionConfig(),))
    pred = parse(output, (ExprExtractionConfig(), LatexExtractionConfig()))
    if not gold or not pred:
        return 0.0
    return 1.0 if any(verify(g, p) for p in pred for g in gold) else 0.0


def compute_score(model_output: str, ground_truth: str, timeout_score: float = 0.0, timeout: float = 30.0, _verify_fn=None) -> float:
    """``_verify_fn`` (tests): a picklable stand-in for the package's verifier, run through the same pool and time-out path."""
    if _verify_fn is None and not available():
        raise ImportError("the math_verify scorer needs the `math-verify` package")
    try:
        return float(_workers().submit(_verify_fn or _verify, "\\boxed{" + str(ground_truth) + "}", model_output).result(timeout=timeout))
    except FuturesTimeout:
        return timeout_score
    except Exception as e:  # noqa: BLE001
        if type(e).__name__ == "TimeoutException":
            return timeout_score
        print(f"Error in math_verify compute_score: {e}")
        return 0.0
