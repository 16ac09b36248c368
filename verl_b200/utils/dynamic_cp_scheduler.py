"""Dynamic context parallelism: choose, per sample, how many ranks share it.

With a fixed context-parallel size every sequence of a micro-batch is cut over all ``cp`` ranks, however short it is. Here a
sample gets the smallest power-of-two number of ranks that keeps its share below ``max_seqlen_per_rank``; short samples run on
one rank with no communication at all, long ones span an aligned sub-group (ranks ``[g·k, (g+1)·k)``), and several samples are
packed onto a group while its per-rank token count allows. Every micro-batch is a list with one entry per rank: the sample ids
that rank works on; ranks with identical lists form one group.

Reference: ``verl/utils/dynamic_cp_scheduler.py:112-286`` — an adapter around Megatron-Core's ``DefaultDynamicCPScheduler``
(``get_groups_and_subsamples``). Megatron-Core is not a dependency here, so the packing itself is implemented below (buddy
allocation of rank groups, first-fit-decreasing placement, idle ranks absorbed by doubling a neighbour group).
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

__all__ = ["DynamicCPScheduler", "local_padding_mask", "cp_members", "postprocess_dynamic_cp_batch"]


def _pow2_at_least(n: int) -> int:
    return 1 << max(0, (int(n) - 1).bit_length())


class _Group:
    __slots__ = ("start", "size", "samples", "tokens")

    def __init__(self, start: int, size: int):
        self.start, self.size, self.samples, self.tokens = start, size, [], 0

    def per_rank(self, extra: int = 0) -> float:
        return (self.tokens + extra) / self.size


class DynamicCPScheduler:
    """``schedule_lengths(seq_lens)`` → micro-batches, each a list of ``total_ranks`` sample-id lists."""

    def __init__(self, max_seqlen_per_dp_cp_rank: int, dp_size: int, cp_size: int):
        if any(type(v) is not int or v <= 0 for v in (max_seqlen_per_dp_cp_rank, dp_size, cp_size)):
            raise ValueError("Dynamic CP scheduler sizes must be positive integers")
        self.max_seqlen_per_dp_cp_rank = max_seqlen_per_dp_cp_rank
        self.dp_size, self.cp_size = dp_size, cp_size
        self.total_ranks = dp_size * cp_size
        if self.total_ranks & (self.total_ranks - 1):
            raise ValueError(f"Dynamic CP needs a power-of-two number of ranks, got {self.total_ranks}")

    # ------------------------------------------------------------------ packing
    def ranks_needed(self, seq_len: int) -> int:
        return _pow2_at_least(math.ceil(seq_len / self.max_seqlen_per_dp_cp_rank))

    def schedule_lengths(self, seq_lens: Sequence[int]) -> list[list[list[int]]]:
        if not len(seq_lens):
            raise ValueError("Dynamic CP cannot schedule an empty batch")
        if any(int(n) <= 0 for n in seq_lens):
            raise ValueError("Dynamic CP requires every input sequence to contain at least one token")
        R, cap = self.total_ranks, self.max_seqlen_per_dp_cp_rank
        need = max(self.ranks_needed(int(n)) for n in seq_lens)
        if need > R:
            raise ValueError(f"A sequence with {max(seq_lens)} tokens needs at least {need} ranks at max_seqlen_per_dp_cp_rank={cap}, "
                             f"but the DPxCP group only has {R} ranks. Increase max_seqlen_per_dp_cp_rank or cap the sequence length.")
        todo = sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i))
        out = []
        while todo:
            groups, free = [], {R: [0]}          # free aligned blocks by size (buddy allocator over the rank axis)
            left = []
            for i in todo:
                n = int(seq_lens[i])
                k = self.ranks_needed(n)
                # first fit into a group of the same width that still has room
                g = next((g for g in groups if g.size == k and g.per_rank(n) <= cap), None)
                if g is None:
                    start = self._take(free, k, R)
                    if start is None:
                        # no block of that width left in this micro-batch. The sample waits for the next one rather than
                        # joining a wider group: being cut over more ranks than it needs is the cost this scheme avoids
                        left.append(i)
                        continue
                    g = _Group(start, k)
                    groups.append(g)
                g.samples.append(i)
                g.tokens += n
            self._absorb_idle(groups, free, seq_lens)
            assign: list[list[int]] = [[] for _ in range(R)]
            for g in groups:
                for r in range(g.start, g.start + g.size):
                    assign[r] = sorted(g.samples)
            out.append(assign)
            todo = left
        return out

    @staticmethod
    def _take(free: dict, k: int, R: int) -> Optional[int]:
        """Lowest-address free block of width k, splitting a wider one when needed."""
        size = k
        while size <= R and not free.get(size):
            size *= 2
        if size > R:
            return None
        start = min(free[size])
        free[size].remove(start)
        while size > k:
            size //= 2
            free.setdefault(size, []).append(start + size)
        return start

    @staticmethod
    def _absorb_idle(groups: list, free: dict, seq_lens) -> None:
        """Idle rank blocks join the buddy group next to them (the group doubles, its per-rank load halves); a group with
        several samples may instead hand one of them to the idle block. What cannot be merged stays idle for this micro-batch."""
        changed = True
        while changed:
            changed = False
            for size in sorted(free):
                for start in sorted(free[size]):
                    buddy = start ^ size
                    g = next((g for g in groups if g.start == buddy and g.size == size), None)
                    if g is not None:
                        free[size].remove(start)
                        g.start, g.size = min(g.start, start), 2 * size
                        changed = True
                        break
                    donor = max((g for g in groups if len(g.samples) > 1 and g.size <= size), key=lambda g: g.per_rank(), default=None)
                    if donor is not None:
                        free[size].remove(start)
                        ng = _Group(start, size)
                        moved = donor.samples.pop()             # its smallest sample (placement went from long to short)
                        ng.samples.append(moved)
                        ng.tokens = int(seq_lens[moved])
                        donor.tokens -= ng.tokens
                        groups.append(ng)
                        changed = True
                        break
                if changed:
                    break

    # ------------------------------------------------------------------ batch front-end
    def schedule(self, seq_lens: Sequence[int], rank: int, *, tp_size: int = 1, cp_layout: str = "zigzag",
                 min_local_rows: Optional[int] = None) -> list[dict]:
        """This rank's micro-batches: ``sample_ids``, ``local_cp_size``, ``cp_rank``, ``members``, ``group_leader``,
        ``padding_mask`` (True on the alignment rows of the local shard) and ``local_num_tokens``. Empty entries (``sample_ids``
        == []) mark micro-batches in which the rank idles."""
        mbs = []
        for assign in self.schedule_lengths(seq_lens):
            ids = assign[rank]
            if not ids:
                mbs.append({"sample_ids": [], "local_cp_size": 1, "cp_rank": 0, "members": [rank], "group_leader": True,
                            "padding_mask": torch.zeros(0, dtype=torch.bool), "local_num_tokens": 0})
                continue
            members = cp_members(assign, rank)
            k = len(members)
            if members != list(range(members[0], members[0] + k)) or members[0] % k:
                raise RuntimeError(f"Dynamic CP group {members} is not an aligned run of ranks")
            mask = local_padding_mask([int(seq_lens[i]) for i in ids], cp_size=k, cp_rank=members.index(rank), tp_size=tp_size,
                                      cp_layout=cp_layout, min_local_rows=min_local_rows)
            mbs.append({"sample_ids": list(ids), "local_cp_size": k, "cp_rank": members.index(rank), "members": members,
                        "group_leader": rank == members[0], "padding_mask": mask, "local_num_tokens": int(mask.numel() - mask.sum())})
        return mbs


def cp_members(rank_assignments: list, rank: int) -> list[int]:
    mine = rank_assignments[rank]
    if not mine:
        raise RuntimeError("empty rank assignment")
    return [p for p, ids in enumerate(rank_assignments) if ids == mine]


def local_padding_mask(seq_lens: Sequence[int], *, cp_size: int, cp_rank: int, tp_size: int, cp_layout: str = "zigzag",
                       min_local_rows: Optional[int] = None) -> torch.Tensor:
    """True on the rows of this rank's shard that are alignment padding (every sequence is padded to a multiple of
    ``tp·cp`` — twice that for the zig-zag layout — before it is cut), False on real tokens."""
    if cp_layout not in ("zigzag", "contiguous"):
        raise ValueError(f"Unsupported context parallel layout: {cp_layout}")
    factor = 2 if cp_layout == "zigzag" and cp_size > 1 else 1
    align = tp_size * cp_size * factor
    padded = [math.ceil(n / align) * align for n in seq_lens]
    if min_local_rows is not None:
        if min_local_rows <= 0:
            raise ValueError(f"min_local_rows must be positive, got {min_local_rows}")
        short = cp_size * min_local_rows - sum(padded)
        if short > 0:
            padded[-1] += short
    if cp_layout == "contiguous":
        tl = sum(padded) // cp_size
        lo, hi = tl * cp_rank, tl * (cp_rank + 1)
        mask = torch.ones(tl, dtype=torch.bool)
        s0 = 0
        for n, p in zip(seq_lens, padded):
            a, b = max(lo, s0), min(hi, s0 + n)
            if a < b:
                mask[a - lo:b - lo] = False
            s0 += p
        return mask
    parts = []
    for n, p in zip(seq_lens, padded):
        m = torch.ones(p // cp_size, dtype=torch.bool)
        if cp_size == 1:
            m[:n] = False
        else:
            half = p // (2 * cp_size)
            front, back = cp_rank * half, p - (cp_rank + 1) * half
            m[: max(0, min(n - front, half))] = False
            m[half: half + max(0, min(n - back, half))] = False
        parts.append(m)
    return torch.cat(parts)


def postprocess_dynamic_cp_batch(output_lst: list, batch_size: int, dcp_group=None, include_model_output: bool = True) -> dict:
    """Collect one output per group (its leader's) from every rank and put the samples back into batch order.
    ``output_lst``: per micro-batch ``{"group_leader", "sample_ids", "loss", "metrics", "model_output": {key: per-sample
    tensors}}``. Returns ``{"model_output": {key: list of per-sample tensors}, "loss": [...], "metrics": {key: [...]}}``."""
    import torch.distributed as dist

    local = []
    for o in output_lst:
        if not o.get("group_leader", False) or not o.get("sample_ids"):
            continue
        ids = [int(i) for i in o["sample_ids"]]
        mo = {}
        for k, v in (o.get("model_output") or {}).items():
            parts = list(v) if isinstance(v, (list, tuple)) else list(v.unbind(0))
            if len(parts) != len(ids):
                raise ValueError(f"Dynamic CP output {k!r} has {len(parts)} samples for ids {ids}")
            mo[k] = [p.detach().cpu() for p in parts]
        local.append({"sample_ids": ids, "loss": o.get("loss"), "metrics": o.get("metrics", {}), "model_output": mo})
    if dcp_group is not None and dist.is_initialized() and dist.get_world_size(dcp_group) > 1:
        gathered = [None] * dist.get_world_size(dcp_group)
        dist.all_gather_object(gathered, local, group=dcp_group)
        records = [r for rs in gathered for r in rs]
    else:
        records = local
    seen = sorted(i for r in records for i in r["sample_ids"])
    if seen != list(range(batch_size)):
        raise RuntimeError(f"Dynamic CP output collection must contain each sample once, got ids {seen}")
    records.sort(key=lambda r: min(r["sample_ids"]))
    by_key: dict = {}
    losses, metrics = [], {}
    for r in records:
        if r["loss"] is not None:
            losses.append(r["loss"])
        for k, v in r["metrics"].items():
            metrics.setdefault(k, []).extend(v if isinstance(v, list) else [v])
        for k, parts in r["model_output"].items():
            d = by_key.setdefault(k, {})
            for i, p in zip(r["sample_ids"], parts):
                d[i] = p
    mo = {}
    if include_model_output:
        for k, d in by_key.items():
            missing = set(range(batch_size)) - set(d)
            if missing:
                raise RuntimeError(f"Dynamic CP output {k!r} is missing sample ids {sorted(missing)}")
            mo[k] = [d[i] for i in range(batch_size)]
    return {"model_output": mo, "loss": losses, "metrics": metrics}
