"""Actor → rollout resharding by kernels that read the trainer ranks' shards in place (NVLink peer loads) and write the
rollout layout directly, optionally re-quantised to block-scaled fp8 in the same pass (``csrc/quant_sync.cu:
reshard_quant_kernel``). The reference materialises full HF tensors on every rank with collectives, ships them through
CUDA-IPC buckets and lets the serving engine re-lay and quantise them (``verl/workers/engine_workers.py:734-836``,
``verl/utils/vllm/vllm_fp8_utils.py``).

A source tensor is described by a pointer table (one entry per trainer rank, from ``SymmetricBuffer.table``) plus its
row-shard geometry; the destination is the row range this rollout rank owns.
"""

from __future__ import annotations

import torch

from verl_b200.ops import _ext

__all__ = ["gather_rows", "gather_rows_fp8", "rollout_row_range"]


def rollout_row_range(total_rows: int, tp_rank: int, tp_size: int) -> tuple[int, int]:
    per = total_rows // tp_size
    return tp_rank * per, per


def _ptrs(ptr_table) -> torch.Tensor:
    t = torch.as_tensor(ptr_table, dtype=torch.int64).cpu().contiguous()
    assert t.dim() == 1
    return t


def gather_rows(ptr_table, rows_per_rank: int, cols: int, row_begin: int, num_rows: int, like: torch.Tensor, ld_src: int = None) -> torch.Tensor:
    """bf16 rows ``[row_begin, row_begin + num_rows)`` of a matrix whose row blocks live on different ranks."""
    _, _, out = _ext.ops().reshard_quant(_ptrs(ptr_table), rows_per_rank, ld_src or cols, row_begin, num_rows, cols, False, True, like)
    return out


def gather_rows_fp8(ptr_table, rows_per_rank: int, cols: int, row_begin: int, num_rows: int, like: torch.Tensor, ld_src: int = None,
                    keep_bf16: bool = False):
    """Same rows as block-scaled fp8: ``(q [num_rows, cols] float8_e4m3fn, scale [ceil(rows/128), ceil(cols/128)], bf16 or None)``."""
    q, s, o = _ext.ops().reshard_quant(_ptrs(ptr_table), rows_per_rank, ld_src or cols, row_begin, num_rows, cols, True, keep_bf16, like)
    return q, s, (o if keep_bf16 else None)
