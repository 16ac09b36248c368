"""Spawned-process worker group: one driver, N worker processes (one per GPU) connected by pipes.

Plays the role of ``RayWorkerGroup`` (``verl/single_controller/ray/base.py:426``) on a single 8-GPU box without Ray:
the launcher exports ``WORLD_SIZE, RANK, LOCAL_RANK, MASTER_ADDR, MASTER_PORT, WG_PREFIX`` into each worker, worker
methods marked with ``@register`` become group-level calls, results come back as futures, several role classes can be
colocated in one process (``create_colocated_worker_cls``), and a watchdog aborts the driver when a worker dies.
"""

from __future__ import annotations

import multiprocessing as mp
import os
import socket
import threading
import traceback
from concurrent.futures import Future
from typing import Any, Optional

from ..base.decorator import MAGIC_ATTR
from ..base.worker import Worker
from ..base.worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup, default_func_generator

__all__ = ["ProcessWorkerGroup", "create_colocated_worker_cls", "WorkerDictSpec"]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class WorkerDictSpec:
    """Picklable description of colocated roles: role name → ClassWithInitArgs."""

    def __init__(self, class_dict: dict[str, ClassWithInitArgs]):
        self.class_dict = class_dict

    def build(self):
        return _build_worker_dict(self.class_dict)


def _build_worker_dict(class_dict: dict[str, ClassWithInitArgs]):
    class WorkerDict(Worker):
        def __init__(self):
            super().__init__()
            self.worker_dict = {}
            for role, cia in class_dict.items():
                self.worker_dict[role] = cia.cls(*cia.args, **cia.kwargs)

    for role, cia in class_dict.items():
        for name in dir(cia.cls):
            try:
                m = getattr(cia.cls, name)
            except Exception:
                continue
            if callable(m) and hasattr(m, MAGIC_ATTR):
                def make(role=role, name=name):
                    def f(self, *a, **k):
                        return getattr(self.worker_dict[role], name)(*a, **k)
                    return f
                fn = make()
                setattr(fn, MAGIC_ATTR, getattr(m, MAGIC_ATTR))
                setattr(WorkerDict, f"{role}_{name}", fn)
    return WorkerDict


def create_colocated_worker_cls(class_dict: dict[str, ClassWithInitArgs]) -> ClassWithInitArgs:
    """Fuse several role classes into one process; methods are exposed as ``<role>_<method>``."""
    spec = WorkerDictSpec(class_dict)
    cia = ClassWithInitArgs(spec)
    cia.is_worker_dict = True
    return cia


def _worker_main(conn, rank: int, world: int, local_rank: int, env: dict, cia: ClassWithInitArgs, use_gpu: bool):
    os.environ.update({k: str(v) for k, v in env.items()})
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(local_rank)})
    try:
        if getattr(cia, "is_worker_dict", False):
            obj = cia.cls.build()()
        else:
            obj = cia()
        conn.send(("ready", None))
    except BaseException as e:  # noqa: BLE001
        conn.send(("error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        return
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            break
        if msg is None:
            break
        call_id, method, args, kwargs = msg
        try:
            out = getattr(obj, method)(*args, **kwargs)
            conn.send((call_id, ("ok", out)))
        except BaseException as e:  # noqa: BLE001
            conn.send((call_id, ("error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}")))


class _WorkerHandle:
    def __init__(self, proc, conn, rank):
        self.proc, self.conn, self.rank = proc, conn, rank
        self.pending: dict[int, Future] = {}
        self.lock = threading.Lock()
        self.next_id = 0
        self.reader = threading.Thread(target=self._read_loop, daemon=True)

    def _read_loop(self):
        while True:
            try:
                call_id, (status, payload) = self.conn.recv()
            except (EOFError, OSError):
                err = RuntimeError(f"worker {self.rank} exited")
                with self.lock:
                    for f in self.pending.values():
                        if not f.done():
                            f.set_exception(err)
                    self.pending.clear()
                return
            with self.lock:
                fut = self.pending.pop(call_id, None)
            if fut is None:
                continue
            if status == "ok":
                fut.set_result(payload)
            else:
                fut.set_exception(RuntimeError(f"worker {self.rank} raised:\n{payload}"))

    def call(self, method, args, kwargs) -> Future:
        fut: Future = Future()
        with self.lock:
            cid = self.next_id
            self.next_id += 1
            self.pending[cid] = fut
        self.conn.send((cid, method, args, kwargs))
        return fut


class ProcessWorkerGroup(WorkerGroup):
    def __init__(self, resource_pool: Optional[ResourcePool] = None, cls_with_init_args: Optional[ClassWithInitArgs] = None,
                 name_prefix: str = "wg", use_gpu: bool = True, env_vars: Optional[dict] = None,
                 worker_handles: Optional[list] = None, bind_cls=None, method_prefix: str = "", start_timeout: float = 600.0,
                 **kwargs):
        super().__init__(resource_pool, **kwargs)
        self.name_prefix = name_prefix
        self.method_prefix = method_prefix
        self.cia = cls_with_init_args
        if worker_handles is not None:   # view on already running workers (spawn of a colocated group)
            self._workers = worker_handles
            self._bind(bind_cls)
            return
        world = resource_pool.world_size
        ctx = mp.get_context("spawn")
        addr, port = "127.0.0.1", str(_free_port())
        self._master_addr, self._master_port = addr, port
        env = {"MASTER_ADDR": addr, "MASTER_PORT": port, "WG_PREFIX": name_prefix, "WG_BACKEND": "process",
               "LOCAL_WORLD_SIZE": str(resource_pool.store[0] if resource_pool.store else world)}
        env.update(env_vars or {})
        local_ranks = resource_pool.local_rank_list()        # for a sub-pool: the parent's device indices of its slice
        for r in range(world):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_worker_main, args=(child, r, world, local_ranks[r], env, cls_with_init_args, use_gpu), daemon=True)
            p.start()
            child.close()
            self._workers.append(_WorkerHandle(p, parent, r))
        for h in self._workers:
            if not h.conn.poll(start_timeout):
                raise TimeoutError(f"worker {h.rank} did not start within {start_timeout} s")
            status, payload = h.conn.recv()
            if status != "ready":
                raise RuntimeError(f"worker {h.rank} failed to start:\n{payload}")
            h.reader.start()
        bind = cls_with_init_args.cls.build() if getattr(cls_with_init_args, "is_worker_dict", False) else cls_with_init_args.cls
        self._bind(bind)

    def _bind(self, cls):
        self._bound_cls = cls
        self._bind_worker_method(cls, self._func_generator)

    def _func_generator(self, wg, method_name, dispatch_fn, collect_fn, execute_fn, blocking):
        return default_func_generator(self, method_name, dispatch_fn, collect_fn, execute_fn, blocking)

    # ------------------------------------------------------------------ execution
    def _is_worker_alive(self, worker: _WorkerHandle) -> bool:
        return worker.proc.is_alive()

    def _wait(self, output):
        return [o.result() if isinstance(o, Future) else o for o in output]

    def execute_all(self, method_name: str, *args, **kwargs):
        n = self.world_size
        futs = []
        for i, h in enumerate(self._workers):
            a = tuple(x[i] for x in args)
            k = {key: v[i] for key, v in kwargs.items()}
            futs.append(h.call(method_name, a, k))
        return futs

    execute_all_async = execute_all

    def execute_all_sync(self, method_name: str, *args, **kwargs):
        return self._wait(self.execute_all(method_name, *args, **kwargs))

    def execute_rank_zero(self, method_name: str, *args, **kwargs):
        return [self._workers[0].call(method_name, args, kwargs)]

    # ------------------------------------------------------------------ colocated roles
    def spawn(self, prefix_set) -> dict[str, "ProcessWorkerGroup"]:
        """Per-role views on a colocated group: ``wg.spawn({"actor", "critic"})["actor"].update_actor(...)``."""
        assert getattr(self.cia, "is_worker_dict", False), "spawn() needs a group built from create_colocated_worker_cls"
        out = {}
        for role in prefix_set:
            role_cls = self.cia.cls.class_dict[role].cls
            view = ProcessWorkerGroup(worker_handles=self._workers, bind_cls=None, name_prefix=self.name_prefix)
            view.cia = self.cia
            view._rebind_role(role, role_cls)
            out[role] = view
        return out

    def _rebind_role(self, role: str, role_cls):
        parent = self

        def gen(wg, method_name, dispatch_fn, collect_fn, execute_fn, blocking):
            def execute_prefixed(name, *a, **k):
                return execute_fn(f"{role}_{name}", *a, **k)
            return default_func_generator(parent, method_name, dispatch_fn, collect_fn, execute_prefixed, blocking)

        self._bind_worker_method(role_cls, gen)

    def shutdown(self):
        for h in self._workers:
            try:
                h.conn.send(None)
            except Exception:
                pass
        for h in self._workers:
            h.proc.join(timeout=5)
            if h.proc.is_alive():
                h.proc.terminate()
