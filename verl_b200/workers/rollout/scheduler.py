"""ctypes front-end of the native continuous-batching scheduler / paged-KV block manager
(``verl_b200/csrc/rollout_scheduler.cpp``). The scheduler is plain host C++ and is also available on CPU-only
machines; a small pure-Python build fallback is *not* provided on purpose — the native library is the product."""

from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch  # noqa: F401  (loads libtorch so the extension's dependencies resolve)

from verl_b200.ops import _ext

__all__ = ["Scheduler", "STEP_IDLE", "STEP_PREFILL", "STEP_DECODE"]

STEP_IDLE, STEP_PREFILL, STEP_DECODE = 0, 1, 2
_lib: Optional[ctypes.CDLL] = None


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _ext.lib_path()
        if not path.exists():
            raise RuntimeError(f"{path} not built; run `python -m verl_b200.csrc.build`")
        lib = ctypes.CDLL(str(path))
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        lib.vb_sched_create.restype = vp
        lib.vb_sched_create.argtypes = [i32, i32, i32, i32, i32]
        lib.vb_sched_destroy.argtypes = [vp]
        lib.vb_sched_add.argtypes = [vp, i64, i32, i32, i64, vp, i32, ctypes.c_uint64]
        lib.vb_sched_step.argtypes = [vp, vp, vp, vp, vp, vp, vp]
        lib.vb_sched_counter.argtypes = [vp, i32]
        lib.vb_sched_counter.restype = i64
        lib.vb_sched_blocks.argtypes = [vp, i64, vp, i32]
        for name in ("vb_sched_num_waiting", "vb_sched_num_running", "vb_sched_num_free_blocks"):
            getattr(lib, name).argtypes = [vp]
        lib.vb_sched_num_preemptions.argtypes = [vp]
        lib.vb_sched_num_preemptions.restype = i64
        for name in ("vb_sched_num_tokens", "vb_sched_num_preempted", "vb_sched_at_limit"):
            getattr(lib, name).argtypes = [vp, i64]
        lib.vb_sched_finish.argtypes = [vp, i64, vp, i32]
        lib.vb_sched_abort_all.argtypes = [vp, vp, i32]
        _lib = lib
    return _lib


class Scheduler:
    """``chunked_prefill``: a prompt longer than ``max_batched_tokens`` is computed in chunks of that size over several prefill
    steps instead of in one oversized step. ``prefix_caching``: full prompt blocks are kept findable by a hash of their
    tokens after their sequence is gone and reused by later sequences that start with the same tokens."""

    def __init__(self, num_blocks: int, block_size: int, max_num_seqs: int, max_batched_tokens: int, chunked_prefill: bool = True,
                 prefix_caching: bool = True):
        self.lib = _load()
        self.h = self.lib.vb_sched_create(num_blocks, block_size, max_num_seqs, max_batched_tokens,
                                          (1 if chunked_prefill else 0) | (2 if prefix_caching else 0))
        self.block_size = block_size
        self.max_num_seqs = max_num_seqs
        cap = max_num_seqs
        self._ids = np.zeros(cap, dtype=np.int64)
        self._slots = np.zeros(cap, dtype=np.int32)
        self._lens = np.zeros(cap, dtype=np.int32)
        self._forks = np.zeros(cap, dtype=np.int64)
        self._starts = np.zeros(cap, dtype=np.int32)
        self.starts = self._starts[:0]
        self._n = ctypes.c_int(0)
        self._blk = np.zeros(4096, dtype=np.int32)

    def __del__(self):
        try:
            if self.h:
                self.lib.vb_sched_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def add(self, seq_id: int, prompt_len: int, max_new_tokens: int, share_key: int = 0, tokens=None, no_chunk: bool = False,
            no_cache: bool = False, salt: int = 0) -> None:
        """``tokens``: the prompt's ids (needed for prefix caching; without them the sequence neither finds nor leaves cached
        blocks). ``salt`` separates prompts whose ids alone do not determine their KV (image placeholders)."""
        tok = None
        if tokens is not None:
            tok = np.ascontiguousarray(tokens, dtype=np.int64)
            assert tok.size >= prompt_len
        rc = self.lib.vb_sched_add(self.h, seq_id, prompt_len, max_new_tokens, share_key, tok.ctypes.data if tok is not None else None,
                                   (1 if no_chunk else 0) | (2 if no_cache or tok is None else 0), salt & 0xFFFFFFFFFFFFFFFF)
        if rc == -1:
            raise ValueError(f"sequence {seq_id} already exists")
        if rc == -2:
            raise ValueError(f"sequence {seq_id} (prompt {prompt_len} + {max_new_tokens}) can never fit the KV cache")

    def step(self):
        """Returns (kind, ids, slots, lens, fork_src) as numpy views valid until the next call. After a prefill step
        ``self.starts[i]`` is the number of prompt tokens of sequence i that are in the cache already (prefix-cache hits or
        earlier chunks): the step computes tokens ``[starts[i], starts[i] + lens[i])``."""
        kind = self.lib.vb_sched_step(self.h, self._ids.ctypes.data, self._slots.ctypes.data, self._lens.ctypes.data,
                                      self._forks.ctypes.data, self._starts.ctypes.data, ctypes.addressof(self._n))
        n = self._n.value
        self.starts = self._starts[:n]
        return kind, self._ids[:n], self._slots[:n], self._lens[:n], self._forks[:n]

    def blocks(self, seq_id: int) -> np.ndarray:
        n = self.lib.vb_sched_blocks(self.h, seq_id, self._blk.ctypes.data, self._blk.size)
        if n < 0:
            raise KeyError(seq_id)
        if n > self._blk.size:
            self._blk = np.zeros(2 * n, dtype=np.int32)
            n = self.lib.vb_sched_blocks(self.h, seq_id, self._blk.ctypes.data, self._blk.size)
        return self._blk[:n].copy()

    def finish(self, seq_id: int, tokens=None) -> None:
        """``tokens``: ids of the leading tokens whose KV this sequence wrote (prompt + generated tokens that were fed back);
        their full blocks stay findable for later prompts."""
        if tokens is None:
            self.lib.vb_sched_finish(self.h, seq_id, None, 0)
            return
        tok = np.ascontiguousarray(tokens, dtype=np.int64)
        self.lib.vb_sched_finish(self.h, seq_id, tok.ctypes.data, int(tok.size))

    @property
    def prefix_cache_hit_tokens(self) -> int:
        return int(self.lib.vb_sched_counter(self.h, 0))

    @property
    def prompt_tokens_admitted(self) -> int:
        return int(self.lib.vb_sched_counter(self.h, 1))

    @property
    def extra_prefill_chunks(self) -> int:
        return int(self.lib.vb_sched_counter(self.h, 2))

    def at_limit(self, seq_id: int) -> bool:
        return self.lib.vb_sched_at_limit(self.h, seq_id) == 1

    def num_tokens(self, seq_id: int) -> int:
        return self.lib.vb_sched_num_tokens(self.h, seq_id)

    def num_preempted(self, seq_id: int) -> int:
        return self.lib.vb_sched_num_preempted(self.h, seq_id)

    def abort_all(self) -> list[int]:
        buf = np.zeros(65536, dtype=np.int64)
        n = self.lib.vb_sched_abort_all(self.h, buf.ctypes.data, buf.size)
        return buf[: min(n, buf.size)].tolist()

    @property
    def num_waiting(self) -> int:
        return self.lib.vb_sched_num_waiting(self.h)

    @property
    def num_running(self) -> int:
        return self.lib.vb_sched_num_running(self.h)

    @property
    def num_free_blocks(self) -> int:
        return self.lib.vb_sched_num_free_blocks(self.h)

    @property
    def num_preemptions(self) -> int:
        return int(self.lib.vb_sched_num_preemptions(self.h))
