"""Actor → rollout resharding by kernels that read the trainer ranks' shards in place (NVLink peer loads) and write the
rollout layout directly, optionally re-quantised to block-scaled fp8 in the same pass (``csrc/quant_sync.cu:
reshard_quant_kernel``). The reference materialises full HF tensors on every rank with collectives, ships them through
CUDA-IPC buckets and lets the serving engine re-lay and quantise them (``verl/workers/engine_workers.py:734-836``,
``verl/utils/vllm/vllm_fp8_utils.py``).

A source tensor is described by a pointer table (one entry per trainer rank, from ``SymmetricBuffer.table``) plus its
row-shard geometry; the destination is the row / column range this rollout rank owns.

:class:`PeerReshardSync` is the product path for trainers whose projection weights are row-sharded in symmetric memory
(the ZeRO-3 mode): every rollout rank fills its own copy — the whole weight, or its tensor-parallel slice cut by the same
rules as :func:`verl_b200.models.parallel_model.shard_param` — with one kernel launch per contiguous block, no collective
and no full-size intermediate. Without the kernels (CPU ranks, weights outside symmetric memory) the same slices are
taken from an all-gathered weight, which is also the oracle of the 2-GPU test.
"""

from __future__ import annotations

import time
from typing import Optional

import torch
import torch.distributed as dist

from verl_b200.ops import _ext

__all__ = ["gather_rows", "gather_rows_fp8", "gather_rows_into", "rollout_row_range", "PeerReshardSync"]


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


def gather_rows_into(ptr_table, rows_per_rank: int, ld_src: int, row_begin: int, out: torch.Tensor, col_begin: int = 0) -> None:
    """Write rows ``[row_begin, row_begin + out.shape[0])``, columns ``[col_begin, col_begin + out.shape[1])`` of the sharded
    matrix into ``out`` (a bf16 view with unit inner stride, e.g. a slice of a parameter) — no allocation."""
    _ext.ops().reshard_into(_ptrs(ptr_table) + 2 * col_begin, rows_per_rank, ld_src, row_begin, out)


class PeerReshardSync:
    """Fills a rollout model (full copy, or the tensor-parallel slice of rank ``tp_rank`` of ``tp``) from a trainer engine
    whose decoder projections are row-sharded over the ranks (``param._zero3``); replicated parameters are plain copies."""

    def __init__(self, engine, target, tp_rank: int = 0, tp: int = 1):
        self.engine, self.target, self.tp_rank, self.tp = engine, target, tp_rank, tp
        self.full_cfg = engine.cfg
        self.last_stats: dict = {}

    # one contiguous block of the FULL weight → the matching block of the destination parameter
    def _block(self, src_param, sh, dst: torch.Tensor, row_begin: int, col_begin: int, full_cache: dict, name: str):
        rows, cols = dst.shape
        fused = (sh.symm is not None and dst.is_cuda and dst.dtype == torch.bfloat16 and _ext.available() and dst.stride(1) == 1
                 and cols % 8 == 0 and col_begin % 8 == 0 and sh.in_features % 8 == 0)
        if fused:
            gather_rows_into(sh.symm.table(sh.byte_offset), sh.rows, sh.in_features, row_begin, dst, col_begin)
            self._peer_bytes += sum(2 * cols * max(0, min(row_begin + rows, (r + 1) * sh.rows) - max(row_begin, r * sh.rows))
                                    for r in range(sh.world) if r != sh.rank)
            return
        full = full_cache.get(name)
        if full is None:                                   # collective fallback: every rank of the shard group takes part
            from verl_b200.workers.engine.fsdp.zero3 import _gather_rows

            full = full_cache[name] = _gather_rows(src_param.data, sh)
        dst.copy_(full[row_begin:row_begin + rows, col_begin:col_begin + cols])

    @torch.no_grad()
    def sync(self) -> dict:
        from verl_b200.models.parallel_model import shard_param, tp_rule

        t0 = time.perf_counter()
        self._peer_bytes = 0
        src = dict(self.engine.model.named_parameters())
        n_kernel = n_copy = 0
        for name, dst in self.target.named_parameters():
            p = src.get(name)
            if p is None:
                continue
            sh = getattr(p, "_zero3", None)
            rule = tp_rule(name, self.full_cfg) if (self.tp > 1 and name.startswith("layers.")) else None
            if sh is None:
                if getattr(p, "_ep_full_shape", None) is not None:
                    from verl_b200.workers.engine.fsdp.zero3 import _gather_dim0

                    full = _gather_dim0(p.data, self.engine.shard_group)
                    dst.copy_(shard_param(name, full, self.full_cfg, self.tp_rank, self.tp) if rule is not None else full)
                elif dst.data_ptr() != p.data_ptr():
                    dst.copy_(shard_param(name, p.data, self.full_cfg, self.tp_rank, self.tp) if rule is not None else p.data)
                n_copy += 1
                continue
            cache: dict = {}
            if rule is None:
                self._block(p, sh, dst, 0, 0, cache, name)
            else:
                dim, segs = rule
                off = dst_off = 0
                for n in segs:
                    per = n // self.tp
                    if dim == 0:
                        self._block(p, sh, dst.narrow(0, dst_off, per), off + self.tp_rank * per, 0, cache, name)
                    else:
                        self._block(p, sh, dst.narrow(1, dst_off, per), 0, off + self.tp_rank * per, cache, name)
                    off += n
                    dst_off += per
            n_kernel += 1
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.last_stats = {"seconds": time.perf_counter() - t0, "sharded_tensors": n_kernel, "replicated_tensors": n_copy,
                           "nvlink_bytes": int(self._peer_bytes)}
        return self.last_stats
