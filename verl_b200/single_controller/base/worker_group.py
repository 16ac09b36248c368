"""Worker-group plumbing shared by all backends: resource pools, deferred class construction, binding of
``@register``-ed worker methods onto the group object, and the liveness watchdog.

Parity target: ``verl/single_controller/base/worker_group.py:27-250``.
"""

from __future__ import annotations

import os
import signal
import threading
import time
from typing import Any, Callable, Optional

from verl_b200.protocol import DataProto, unpad_dataproto

from .decorator import MAGIC_ATTR, Dispatch, get_predefined_dispatch_fn, get_predefined_execute_fn

__all__ = ["ResourcePool", "SubResourcePool", "ResourcePoolManager", "split_resource_pool", "merge_resource_pool", "ClassWithInitArgs", "WorkerGroup"]


class ResourcePool:
    """``process_on_nodes[i]`` worker processes (one per GPU) on node i."""

    def __init__(self, process_on_nodes=None, max_colocate_count: int = 10, n_gpus_per_node: int = 8) -> None:
        self._store = list(process_on_nodes or [])
        self.max_colocate_count = max_colocate_count
        self.n_gpus_per_node = n_gpus_per_node

    def add_node(self, process_count: int):
        self._store.append(process_count)

    @property
    def world_size(self) -> int:
        return sum(self._store)

    def __call__(self) -> list[int]:
        return self._store

    @property
    def store(self) -> list[int]:
        return self._store

    def local_world_size_list(self) -> list[int]:
        return [n for n in self._store for _ in range(n)]

    def local_rank_list(self) -> list[int]:
        return [i for n in self._store for i in range(n)]

    def device_slots(self) -> list[tuple[int, int]]:
        """(node index, device index on that node) of every worker of this pool, in rank order."""
        return [(node, i) for node, n in enumerate(self._store) for i in range(n)]


class SubResourcePool(ResourcePool):
    """A contiguous slice of a parent pool's device slots (reference: ``SubRayResourcePool``,
    ``verl/single_controller/ray/base.py:170-186``): worker ``i`` of a group built on it runs on the parent's slot
    ``start_index + i``, so several groups can own disjoint GPUs of one machine."""

    def __init__(self, parent: ResourcePool, start_index: int, size: int):
        super().__init__(parent.store, parent.max_colocate_count, parent.n_gpus_per_node)
        assert 0 <= start_index and start_index + size <= len(parent.device_slots()), "slice exceeds the parent pool"
        self.parent, self.start_index, self.size = parent, start_index, size

    @property
    def world_size(self) -> int:
        return self.size

    def device_slots(self) -> list[tuple[int, int]]:
        return self.parent.device_slots()[self.start_index:self.start_index + self.size]

    def local_rank_list(self) -> list[int]:
        return [d for _, d in self.device_slots()]

    def local_world_size_list(self) -> list[int]:
        slots = self.device_slots()
        per_node: dict = {}
        for node, _ in slots:
            per_node[node] = per_node.get(node, 0) + 1
        return [per_node[node] for node, _ in slots]


def split_resource_pool(pool: ResourcePool, split_size) -> list:
    """Cut ``pool`` into sub-pools of ``split_size`` workers each (an int that divides the world size, or a list of sizes
    that sums to it). Sub-pools can be split again (reference: ``verl/single_controller/ray/base.py:280-327``)."""
    if isinstance(split_size, int):
        assert split_size > 0 and pool.world_size % split_size == 0, "split_size must be a divisor of world_size"
        sizes = [split_size] * (pool.world_size // split_size)
    else:
        sizes = list(split_size)
    assert sum(sizes) == pool.world_size, "split sizes must sum up to world_size"
    out, start = [], 0
    for n in sizes:
        out.append(SubResourcePool(pool, start, n))
        start += n
    return out


def merge_resource_pool(a: ResourcePool, b: ResourcePool) -> ResourcePool:
    """One pool over the nodes of both (``a``'s nodes first); both must agree on colocation and GPUs per node
    (reference: ``verl/single_controller/ray/base.py:329-345``)."""
    assert a.max_colocate_count == b.max_colocate_count, "both pools must have the same max_colocate_count"
    assert a.n_gpus_per_node == b.n_gpus_per_node, "both pools must have the same n_gpus_per_node"
    assert not isinstance(a, SubResourcePool) and not isinstance(b, SubResourcePool), "merge whole pools, not slices"
    return ResourcePool(list(a.store) + list(b.store), a.max_colocate_count, a.n_gpus_per_node)


class ResourcePoolManager:
    """Named pools and a role → pool mapping: ``resource_pool_spec = {"global_pool": [8, 8]}``, ``mapping = {"actor_rollout":
    "global_pool", "critic": "global_pool"}`` (reference: ``verl/single_controller/ray/base.py:189-247``). ``available`` is
    the number of devices this launcher can place workers on (default: what ``torch.cuda.device_count()`` reports, or no
    limit on CPU); creation fails early when the spec asks for more."""

    def __init__(self, resource_pool_spec: dict, mapping: dict, max_colocate_count: int = 3, available: Optional[int] = None):
        self.resource_pool_spec, self.mapping, self.max_colocate_count = dict(resource_pool_spec), dict(mapping), max_colocate_count
        self.available = available
        self.resource_pool_dict: dict = {}

    def create_resource_pool(self):
        for name, process_on_nodes in self.resource_pool_spec.items():
            self.resource_pool_dict[name] = ResourcePool(list(process_on_nodes), self.max_colocate_count)
        self._check_resource_available()
        return self.resource_pool_dict

    def get_resource_pool(self, role) -> ResourcePool:
        return self.resource_pool_dict[self.mapping[role]]

    def get_n_gpus(self) -> int:
        return sum(n for nodes in self.resource_pool_spec.values() for n in nodes)

    def _check_resource_available(self):
        have = self.available
        if have is None:
            try:
                import torch

                have = torch.cuda.device_count() if torch.cuda.is_available() else None
            except Exception:  # noqa: BLE001
                have = None
        if have is None:
            return
        total = self.get_n_gpus()
        single_node = all(len(nodes) == 1 for nodes in self.resource_pool_spec.values())
        if single_node and total > have:
            raise ValueError(f"Total available devices {have} is less than total desired devices {total}")
        if any(n > have for nodes in self.resource_pool_spec.values() for n in nodes):
            raise ValueError(f"a pool asks for more devices on one node than the {have} a node has")


class ClassWithInitArgs:
    """A class plus constructor arguments, instantiated later inside the worker process."""

    def __init__(self, cls, *args, **kwargs) -> None:
        self.cls = cls
        self.args = args
        self.kwargs = kwargs
        self.fused_worker_used = False

    def __call__(self) -> Any:
        return self.cls(*self.args, **self.kwargs)


def _check_workers_alive(workers: list, is_alive: Callable, gap_time: float = 1.0) -> None:
    main_pid = os.getpid()
    while True:
        for w in workers:
            if not is_alive(w):
                print(f"worker {w} is not alive; sending SIGABRT to the controller process {main_pid}", flush=True)
                os.kill(main_pid, signal.SIGABRT)
                return
        time.sleep(gap_time)


class WorkerGroup:
    fused_worker_execute_fn_name = "_fuw_execute"

    def __init__(self, resource_pool: Optional[ResourcePool] = None, **kwargs) -> None:
        self._is_init_with_detached_workers = resource_pool is None
        self.fused_worker_used = False
        self._procs_per_node = resource_pool.store if resource_pool is not None else None
        self._workers: list = []
        self._worker_names: list = []
        self._dispatch_info: dict[str, list[int]] = {}
        self._collect_info: dict[str, list[bool]] = {}
        self._master_addr = None
        self._master_port = None
        self._checker_thread: Optional[threading.Thread] = None

    # ------------------------------------------------------------------ liveness
    def _is_worker_alive(self, worker) -> bool:
        raise NotImplementedError

    def _block_until_all_workers_alive(self) -> None:
        while not all(self._is_worker_alive(w) for w in self._workers):
            time.sleep(0.1)

    def start_worker_aliveness_check(self, every_n_seconds: float = 1.0) -> None:
        """Daemon thread that aborts the controller (SIGABRT) as soon as any worker process has died."""
        self._block_until_all_workers_alive()
        self._checker_thread = threading.Thread(target=_check_workers_alive, args=(self._workers, self._is_worker_alive, every_n_seconds), daemon=True)
        self._checker_thread.start()

    @property
    def world_size(self) -> int:
        return len(self._workers)

    # ------------------------------------------------------------------ n-d mesh info
    def query_dispatch_info(self, mesh_name: str) -> list[int]:
        if mesh_name not in self._dispatch_info:
            self._dispatch_info[mesh_name] = self._query_dispatch_info(mesh_name)
        return self._dispatch_info[mesh_name]

    def query_collect_info(self, mesh_name: str) -> list[bool]:
        if mesh_name not in self._collect_info:
            self._collect_info[mesh_name] = self._query_collect_info(mesh_name)
        return self._collect_info[mesh_name]

    # ------------------------------------------------------------------ method binding
    def _bind_worker_method(self, user_defined_cls, func_generator) -> list[str]:
        """For every ``@register``-ed method of the worker class create ``self.<name>(*args)`` that dispatches the
        arguments, runs the method on the workers and collects the results."""
        names = []
        for method_name in dir(user_defined_cls):
            try:
                method = getattr(user_defined_cls, method_name)
                assert callable(method)
            except Exception:
                continue
            if not hasattr(method, MAGIC_ATTR):
                continue
            attrs = getattr(method, MAGIC_ATTR)
            dispatch_mode, execute_mode, blocking = attrs["dispatch_mode"], attrs["execute_mode"], attrs["blocking"]
            if isinstance(dispatch_mode, Dispatch):
                fns = get_predefined_dispatch_fn(dispatch_mode)
            else:
                fns = dispatch_mode
            execute_fn = getattr(self, get_predefined_execute_fn(execute_mode)["execute_fn_name"])
            func = func_generator(self, method_name, dispatch_fn=fns["dispatch_fn"], collect_fn=fns["collect_fn"],
                                  execute_fn=execute_fn, blocking=blocking)
            try:
                setattr(self, method_name, func)
                names.append(method_name)
            except Exception as e:
                raise ValueError(f"failed to bind method {method_name}") from e
        return names

    # to be provided by backends
    def execute_all(self, method_name: str, *args, **kwargs):
        raise NotImplementedError

    def execute_rank_zero(self, method_name: str, *args, **kwargs):
        raise NotImplementedError


def default_func_generator(self: WorkerGroup, method_name: str, dispatch_fn, collect_fn, execute_fn, blocking: bool):
    """dispatch → execute → (wait) → collect, with auto-padding undone after the collect."""

    def func(*args, **kwargs):
        args, kwargs = dispatch_fn(self, *args, **kwargs)
        pad = kwargs.pop("_pad_size", None) if isinstance(kwargs, dict) else None
        output = execute_fn(method_name, *args, **kwargs)
        if blocking:
            output = self._wait(output)
        output = collect_fn(self, output)
        if pad and isinstance(output, DataProto):
            output = unpad_dataproto(output, pad)
        return output

    func.__name__ = method_name
    return func
