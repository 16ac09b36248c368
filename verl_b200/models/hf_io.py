"""HuggingFace checkpoint interop: sharded safetensors read/write with HF tensor names.

The reference delegates this to ``transformers`` ``from_pretrained`` / ``save_pretrained``
(``verl/utils/checkpoint/fsdp_checkpoint_manager.py:138-192``); here tensors are streamed shard by shard so a model
never has to exist twice in host memory.
"""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Iterable, Iterator

import torch

__all__ = ["load_hf_weights", "iter_safetensors", "save_hf_weights", "save_hf_checkpoint", "MAX_SHARD_BYTES"]

MAX_SHARD_BYTES = 5 * 1024**3


def iter_safetensors(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    """Yield (name, tensor) from every ``*.safetensors`` file of a model directory (index-aware)."""
    from safetensors import safe_open

    p = Path(path)
    index = p / "model.safetensors.index.json"
    if index.exists():
        files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    else:
        files = sorted(f.name for f in p.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    for fn in files:
        with safe_open(str(p / fn), framework="pt", device="cpu") as f:
            for k in f.keys():
                yield k, f.get_tensor(k)


def load_hf_weights(model, path: str, strict: bool = True) -> None:
    sd = dict(iter_safetensors(path))
    model.load_hf_state_dict(sd, strict=strict)


def save_hf_weights(named_tensors: Iterable[tuple[str, torch.Tensor]], path: str, dtype: torch.dtype = torch.bfloat16,
                    max_shard_bytes: int = MAX_SHARD_BYTES) -> list[str]:
    """Stream tensors into ``model-0000i-of-0000n.safetensors`` shards (≤ ``max_shard_bytes``) + index json."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    shards: list[dict[str, torch.Tensor]] = [{}]
    sizes = [0]
    for name, t in named_tensors:
        t = t.detach().to(dtype=dtype, device="cpu").contiguous().clone()
        nbytes = t.numel() * t.element_size()
        if sizes[-1] > 0 and sizes[-1] + nbytes > max_shard_bytes:
            shards.append({})
            sizes.append(0)
        shards[-1][name] = t
        sizes[-1] += nbytes
    n = len(shards)
    weight_map, files = {}, []
    for i, sh in enumerate(shards):
        fn = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
        save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
        files.append(fn)
        for k in sh:
            weight_map[k] = fn
    if n > 1:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": sum(sizes)}, "weight_map": weight_map}, f, indent=2)
    return files


def save_hf_checkpoint(model, path: str, dtype: torch.dtype = torch.bfloat16) -> None:
    """``config.json`` + safetensors shards of a ``DecoderLM`` in HuggingFace layout (loadable by ``transformers``)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(model.cfg.to_hf_dict(), f, indent=2)
    save_hf_weights(model.hf_named_tensors(), path, dtype=dtype)
