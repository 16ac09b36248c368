"""Helpers shared by the training engines (reference: ``verl/workers/engine/utils.py``): micro-batch preparation,
output post-processing, determinism switches."""

from __future__ import annotations

import os
import random
from typing import Any

import numpy as np
import torch

from verl_b200.protocol import DataProto
from verl_b200.utils.seqlen_balancing import rearrange_micro_batches, restore_dynamic_batch

__all__ = ["prepare_micro_batches", "postprocess_batch_func", "detach_tree", "enable_full_determinism", "set_seed"]


def prepare_micro_batches(data: DataProto, dp_group=None, same_micro_num_in_dp: bool = True, sp_size: int = 1):
    """→ (list of micro-batch DataProtos, index lists). Dynamic batching packs sequences up to
    ``max_token_len_per_gpu · sp_size`` tokens; otherwise fixed ``micro_batch_size_per_gpu`` rows."""
    meta = data.meta_info
    n = len(data)
    if meta.get("use_dynamic_bsz", False):
        seq_lens = data.batch["attention_mask"].sum(-1)
        idx = rearrange_micro_batches(seq_lens.cpu(), int(meta["max_token_len_per_gpu"]) * sp_size,
                                      dp_group=dp_group if same_micro_num_in_dp else None)
    else:
        mbs = int(meta.get("micro_batch_size_per_gpu", 0) or n)
        idx = [list(range(i, min(n, i + mbs))) for i in range(0, n, mbs)]
    return [data[torch.as_tensor(ix, dtype=torch.int64)] for ix in idx], idx


def postprocess_batch_func(outputs: list[dict], indices: list[list[int]]) -> dict:
    """Concatenate per-micro-batch output dicts and undo the dynamic-batch permutation."""
    keys = outputs[0].keys() if outputs else []
    return {k: restore_dynamic_batch(torch.cat([o[k] for o in outputs], 0), indices) for k in keys}


def detach_tree(x: Any) -> Any:
    if isinstance(x, torch.Tensor):
        return x.detach()
    if isinstance(x, dict):
        return {k: detach_tree(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(detach_tree(v) for v in x)
    return x


def set_seed(seed: int):
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def enable_full_determinism(seed: int = 0):
    """Bitwise reproducible runs: fixed seeds, deterministic library algorithms, ring/simple NCCL so reduction order is
    fixed, and this framework's own kernels in their deterministic variants (split-K off, atomics-free attention dq)."""
    set_seed(seed)
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    os.environ["NCCL_ALGO"] = "Ring"
    os.environ["NCCL_PROTO"] = "Simple"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["VERL_B200_DETERMINISTIC"] = "1"
    torch.use_deterministic_algorithms(True, warn_only=True)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
