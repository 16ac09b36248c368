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

__all__ = ["ResourcePool", "ClassWithInitArgs", "WorkerGroup"]


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
