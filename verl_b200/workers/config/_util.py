"""Helpers shared by the typed config modules."""

from __future__ import annotations

import dataclasses
from dataclasses import field

__all__ = ["from_config", "_sub"]


def from_config(cls, node, **extra):
    """Build ``cls`` from a yaml node (dict-like), recursing into fields whose default is itself a config dataclass.
    Unknown keys of the node are ignored, so a yaml tree may carry more than a class models."""
    if node is None:
        return cls(**extra)
    if isinstance(node, cls):
        return node
    kw = {}
    for f in dataclasses.fields(cls):
        if f.name.startswith("_") or f.name not in node:
            continue
        v = node[f.name]
        sub = f.metadata.get("cls")
        if sub is not None and v is not None and not isinstance(v, sub):
            v = from_config(sub, v)
        elif hasattr(v, "items") and not dataclasses.is_dataclass(v):
            v = dict(v)
        elif isinstance(v, (list, tuple)):
            v = list(v)
        kw[f.name] = v
    kw.update(extra)
    return cls(**kw)


def _sub(cls):
    return field(default_factory=cls, metadata={"cls": cls})
