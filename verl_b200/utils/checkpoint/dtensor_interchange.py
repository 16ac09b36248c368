"""Reading and writing the reference's sharded FSDP model files (``model_world_size_{W}_rank_{r}.pt`` holding DTensors).

The reference saves, per rank, a plain dict ``{HF parameter name: DTensor}`` whose local tensors are dim-0 shards over an
``("fsdp",)`` mesh (or ``("ddp", "fsdp")`` under HSDP: replicated over the first dimension); buffers and unsharded entries are
plain tensors identical on every rank (``verl/utils/checkpoint/fsdp_checkpoint_manager.py:296-330``; merged by
``verl/model_merger/fsdp_model_merger.py:53-253``). This engine keeps one flat buffer per rank instead, so interchange goes
through full HF-named tensors:

* ``merge_sharded_model_files`` rebuilds ``{name: full tensor}`` from such a directory — no process group is needed, the local
  tensors, placements and mesh of an unpickled DTensor are enough;
* ``dtensor_model_payload`` cuts this rank's dim-0 piece of every HF tensor (``ceil(n/W)`` rows per rank, the trailing ranks may
  hold fewer or none — the same rule ``torch.chunk`` and FSDP2 use) and wraps it as a DTensor on a mesh over the running group, so
  that the reference's merger and loader accept the file.

Optimizer state is not interchanged: the reference stores per-parameter ``torch.optim.AdamW`` state, this engine one flat fp32
master / moment slice per rank; a checkpoint of the other format loads weights only and restarts the moments.
"""

from __future__ import annotations

import json
import os
import re
from typing import Iterable, Optional

import torch

__all__ = ["is_named_tensor_payload", "merge_sharded_model_files", "dtensor_model_payload", "saved_world_size"]


def _dtensor_cls():
    from torch.distributed.tensor import DTensor

    return DTensor


def is_named_tensor_payload(obj) -> bool:
    """True for the reference's model files (a dict of tensors), False for this engine's ``flat_v1`` payload."""
    return isinstance(obj, dict) and "format" not in obj and len(obj) > 0 and all(isinstance(v, torch.Tensor) for v in obj.values())


def saved_world_size(local_dir: str) -> int:
    cfg = os.path.join(local_dir, "fsdp_config.json")
    if os.path.exists(cfg):
        with open(cfg) as f:
            w = json.load(f).get("world_size")
        if w:
            return int(w)
    sizes = {int(m.group(1)) for fn in os.listdir(local_dir) if (m := re.match(r"model_world_size_(\d+)_rank_\d+\.pt$", fn))}
    if len(sizes) != 1:
        raise FileNotFoundError(f"cannot tell the world size of the checkpoint in {local_dir} (found {sorted(sizes)})")
    return sizes.pop()


def merge_sharded_model_files(local_dir: str, world_size: Optional[int] = None, dtype: Optional[torch.dtype] = None) -> dict:
    """``{name: full tensor}`` from the per-rank files of ``local_dir``."""
    DTensor = _dtensor_cls()
    W = world_size or saved_world_size(local_dir)
    load = lambda r: torch.load(os.path.join(local_dir, f"model_world_size_{W}_rank_{r}.pt"), map_location="cpu", weights_only=False)  # noqa: E731
    first = load(0)
    if not is_named_tensor_payload(first):
        raise ValueError("not a named-tensor (DTensor) checkpoint")
    pivot = next((v for v in first.values() if isinstance(v, DTensor)), None)
    n_shards, drop = W, 0
    if pivot is not None:
        names = tuple(pivot.device_mesh.mesh_dim_names or ())
        names = ("fsdp",) if names in (("dp_shard",), ()) else names
        if names not in (("fsdp",), ("ddp", "fsdp")):
            raise NotImplementedError(f"unsupported device mesh {names}")
        n_shards = int(pivot.device_mesh.mesh.shape[-1])
        drop = len(names) - 1                    # leading replicate dimension of an HSDP mesh: the first fsdp group has everything
    shards = [first] + [load(r) for r in range(1, n_shards)]
    out = {}
    for key in first:
        vals = [s[key] for s in shards]
        if isinstance(vals[0], DTensor):
            placements = tuple(vals[0].placements)[drop:]
            if len(placements) != 1:
                raise NotImplementedError(f"{key}: placements {vals[0].placements} are not a plain fsdp sharding")
            pl = placements[0]
            locs = [v._local_tensor for v in vals]
            if pl.is_replicate():
                full = locs[0]
            elif pl.is_shard():
                full = torch.cat(locs, dim=pl.dim).contiguous()
            else:
                raise NotImplementedError(f"{key}: unsupported placement {pl}")
            if tuple(full.shape) != tuple(vals[0].shape):
                raise ValueError(f"{key}: merged shape {tuple(full.shape)} differs from the recorded global shape {tuple(vals[0].shape)}")
        else:
            for r, v in enumerate(vals[1:], start=1):
                if v.shape != vals[0].shape or not torch.equal(v, vals[0]):
                    raise ValueError(f"plain entry {key!r} differs between rank 0 and rank {r}: expected a replicated tensor")
            full = vals[0]
        out[key] = full.to(dtype) if dtype is not None and full.is_floating_point() else full
    return out


def dtensor_model_payload(named_tensors: Iterable, rank: int, world: int, fsdp_size: Optional[int] = None, device_type: str = "cpu") -> dict:
    """This rank's file content in the reference's form. ``named_tensors``: (HF name, full tensor) pairs available on every rank.
    ``world == 1`` writes plain tensors (what FSDP produces without sharding). ``fsdp_size < world``: an HSDP mesh ("ddp", "fsdp")."""
    if world == 1:
        return {k: v.detach().to("cpu", copy=True) for k, v in named_tensors}
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Replicate, Shard

    F = int(fsdp_size or world)
    if world % F:
        raise ValueError(f"fsdp_size {F} does not divide the world size {world}")
    if F == world:
        mesh, placements = init_device_mesh(device_type, (world,), mesh_dim_names=("fsdp",)), [Shard(0)]
    else:
        mesh, placements = init_device_mesh(device_type, (world // F, F), mesh_dim_names=("ddp", "fsdp")), [Replicate(), Shard(0)]
    fr = rank % F
    out = {}
    for k, v in named_tensors:
        v = v.detach()
        if v.dim() == 0:
            out[k] = v.to("cpu", copy=True)
            continue
        n = v.shape[0]
        per = -(-n // F)
        lo, hi = min(n, fr * per), min(n, (fr + 1) * per)
        loc = v[lo:hi].to("cpu", copy=True).contiguous() if device_type == "cpu" else v[lo:hi].clone().contiguous()
        out[k] = DTensor.from_local(loc, mesh, placements, run_check=False, shape=v.shape, stride=tuple(v.contiguous().stride()))
    return out
