"""Small pure-Python helpers (reference: ``verl/utils/py_functional.py``)."""

from __future__ import annotations

import contextlib
import os
from typing import Any, Iterable

__all__ = ["append_to_dict", "union_two_dict", "temp_env_var", "DynamicEnum", "convert_to_regular_types", "rename_dict", "timeout_limit"]


def append_to_dict(data: dict, new_data: dict, prefix: str = ""):
    for k, v in new_data.items():
        data.setdefault(prefix + k, []).append(v)


def union_two_dict(a: dict, b: dict) -> dict:
    for k, v in b.items():
        if k in a:
            assert a[k] == v, f"{k} in both dicts with different values"
        a[k] = v
    return a


def rename_dict(d: dict, prefix: str = "") -> dict:
    return {prefix + k: v for k, v in d.items()}


@contextlib.contextmanager
def temp_env_var(key: str, value: str):
    old = os.environ.get(key)
    os.environ[key] = value
    try:
        yield
    finally:
        if old is None:
            os.environ.pop(key, None)
        else:
            os.environ[key] = old


class DynamicEnumMeta(type):
    def __iter__(cls):
        return iter(cls._registry.values())

    def __contains__(cls, item):
        return item in cls._registry or item in cls._registry.values()

    def __getitem__(cls, name):
        return cls._registry[name]


class DynamicEnum(metaclass=DynamicEnumMeta):
    """An enum that can gain members at run time (``Cls.register("NAME")``); used for registries of estimators."""

    _registry: dict[str, "DynamicEnum"] = {}
    _next_value = 0

    def __init_subclass__(cls, **kw):
        cls._registry, cls._next_value = {}, 0

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __repr__(self):
        return f"<{type(self).__name__}.{self.name}: {self.value}>"

    @classmethod
    def register(cls, name: str):
        key = name.upper()
        if key in cls._registry:
            raise ValueError(f"{key} already registered")
        m = cls(key, cls._next_value)
        cls._registry[key] = m
        setattr(cls, key, m)
        cls._next_value += 1
        return m

    @classmethod
    def remove(cls, name: str):
        m = cls._registry.pop(name.upper())
        delattr(cls, name.upper())
        return m

    @classmethod
    def from_name(cls, name: str):
        return cls._registry.get(name.upper())


def convert_to_regular_types(obj: Any) -> Any:
    """Config containers → plain dict / list (for JSON dumps)."""
    if hasattr(obj, "items"):
        return {k: convert_to_regular_types(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [convert_to_regular_types(v) for v in obj]
    return obj


@contextlib.contextmanager
def timeout_limit(seconds: float):
    """Raise ``TimeoutError`` in the main thread if the body runs longer than ``seconds`` (SIGALRM; no-op elsewhere)."""
    import signal
    import threading

    if threading.current_thread() is not threading.main_thread() or seconds is None or seconds <= 0:
        yield
        return

    def handler(signum, frame):
        raise TimeoutError(f"operation exceeded {seconds}s")

    old = signal.signal(signal.SIGALRM, handler)
    signal.setitimer(signal.ITIMER_REAL, seconds)
    try:
        yield
    finally:
        signal.setitimer(signal.ITIMER_REAL, 0)
        signal.signal(signal.SIGALRM, old)
