"""Dynamic import helpers (reference: ``verl/utils/import_utils.py``)."""

from __future__ import annotations

import importlib
import importlib.util
import os
import warnings
from functools import cache, wraps


@cache
def is_package_available(name: str) -> bool:
    return importlib.util.find_spec(name) is not None


def load_extern_type(file_path: str, type_name: str):
    """Load ``type_name`` from a python file given by path (``pkg://module.path`` loads an importable module)."""
    if file_path.startswith("pkg://"):
        module = importlib.import_module(file_path[len("pkg://"):])
    else:
        if file_path.startswith("file://"):
            file_path = file_path[len("file://"):]
        if not os.path.exists(file_path):
            raise FileNotFoundError(f"Custom type file '{file_path}' not found.")
        spec = importlib.util.spec_from_file_location("custom_module", file_path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
    if not hasattr(module, type_name):
        raise AttributeError(f"Custom type '{type_name}' not found in '{file_path}'.")
    return getattr(module, type_name)


def load_class_from_fqn(fqn: str, description: str = "class"):
    mod, _, name = fqn.rpartition(".")
    try:
        return getattr(importlib.import_module(mod), name)
    except (ImportError, AttributeError) as e:
        raise ImportError(f"cannot load {description} '{fqn}': {e}") from e


def deprecated(replacement: str = ""):
    def deco(obj):
        msg = f"{obj.__name__} is deprecated" + (f"; use {replacement}" if replacement else "")

        @wraps(obj)
        def inner(*a, **k):
            warnings.warn(msg, FutureWarning, stacklevel=2)
            return obj(*a, **k)

        return inner

    return deco
