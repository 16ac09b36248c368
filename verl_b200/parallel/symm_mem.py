"""Symmetric memory over NVLink: every rank allocates the same buffer, exports it with CUDA IPC and maps all peers'
copies, so device code can load/store any rank's memory directly.

This is the transport under the fused compute+collective kernels (``verl_b200/csrc/symm_comm.cu`` and the fused GEMM
epilogues). Handles travel through the process group's host (gloo) side once at allocation; afterwards no host library
is involved in the data path. NCCL remains the baseline and the fallback.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from verl_b200.ops import _ext

__all__ = ["SymmetricBuffer", "symm_available"]


def symm_available(group=None) -> bool:
    return torch.cuda.is_available() and dist.is_initialized() and _ext.available()


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group`` plus a small signal pad for device-side barriers."""

    PAD_BYTES = 4096

    def __init__(self, nbytes: int, group=None, host_group=None):
        self.ops = _ext.ops()
        self.group = group if group is not None else dist.group.WORLD
        self.host_group = host_group if host_group is not None else self.group
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.nbytes = int(-(-nbytes // 256) * 256)
        self.local_ptr = int(self.ops.symm_alloc(self.nbytes + self.PAD_BYTES))
        handle = self.ops.ipc_get_handle(self.local_ptr)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.numpy().tobytes(), group=self.host_group)
        self.peer_ptrs = []
        self._opened = []
        for r, hb in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
            else:
                p = int(self.ops.ipc_open_handle(torch.frombuffer(bytearray(hb), dtype=torch.uint8)))
                self._opened.append(p)
                self.peer_ptrs.append(p)
        self.ptr_table = torch.tensor(self.peer_ptrs, dtype=torch.int64)
        self.pad_table = torch.tensor([p + self.nbytes for p in self.peer_ptrs], dtype=torch.int64)
        self.epoch = 0
        dist.barrier(group=self.host_group)

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, byte_offset: int = 0) -> torch.Tensor:
        """View of the *local* copy."""
        es = torch.empty(0, dtype=dtype).element_size()
        n = (self.nbytes - byte_offset) // es if numel is None else numel
        assert byte_offset + n * es <= self.nbytes
        return self.ops.tensor_from_ptr(self.local_ptr + byte_offset, [n], dtype)

    def table(self, byte_offset: int = 0) -> torch.Tensor:
        """CPU int64 tensor of every rank's pointer to ``byte_offset`` inside the buffer."""
        return self.ptr_table + byte_offset

    def barrier(self):
        """Device-side barrier on the current stream (bounded wait; failures surface through ``check_status``)."""
        self.epoch += 1
        self.ops.symm_barrier(self.pad_table, self.rank, self.world, self.epoch)

    def barrier_auto(self):
        """Same, with the epoch counted on the device: safe to capture into a CUDA graph and replay."""
        self.ops.symm_barrier_auto(self.pad_table, self.rank, self.world)

    def close(self):
        for p in self._opened:
            self.ops.ipc_close(p)
        self._opened = []
        if self.local_ptr:
            self.ops.symm_free(self.local_ptr)
            self.local_ptr = 0
