"""``@register`` — turns a worker method into a group-level call with a dispatch (how arguments are split over
workers) and a collect (how results are merged) policy.

Parity target: ``verl/single_controller/base/decorator.py`` (Dispatch/Execute :26-68, dispatch functions :120-304,
n-d mesh dispatch :308-355, register :398-444).
"""

from __future__ import annotations

import inspect
from enum import Enum
from functools import partial, wraps
from typing import Callable

from verl_b200.protocol import DataProto, DataProtoFuture, pad_dataproto_to_divisor, unpad_dataproto

__all__ = ["Dispatch", "Execute", "register", "get_predefined_dispatch_fn", "get_predefined_execute_fn",
           "register_dispatch_mode", "update_dispatch_mode", "make_nd_compute_dataproto_dispatch_fn", "MAGIC_ATTR"]

MAGIC_ATTR = "attrs_3141562937"


class _DynamicEnum:
    """Enum-like registry that can grow at run time (user dispatch modes)."""

    _registry: dict
    _next: int

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __repr__(self):
        return f"<{type(self).__name__}.{self.name}: {self.value}>"

    def __eq__(self, other):
        return type(other) is type(self) and other.value == self.value

    def __hash__(self):
        return hash((type(self).__name__, self.value))

    @classmethod
    def register(cls, name: str):
        key = name.upper()
        if key in cls._registry:
            raise ValueError(f"{key} already registered")
        obj = cls(key, cls._next)
        cls._registry[key] = obj
        setattr(cls, key, obj)
        cls._next += 1
        return obj

    @classmethod
    def remove(cls, name: str):
        key = name.upper()
        obj = cls._registry.pop(key)
        delattr(cls, key)
        return obj

    @classmethod
    def from_name(cls, name: str):
        return cls._registry.get(name.upper())


class Dispatch(_DynamicEnum):
    _registry = {}
    _next = 0


for _n in ("RANK_ZERO", "ONE_TO_ALL", "ALL_TO_ALL", "DP_COMPUTE", "DP_COMPUTE_PROTO", "DP_COMPUTE_PROTO_WITH_FUNC",
           "DP_COMPUTE_METRIC", "DIRECT_ROLLOUT_METHOD"):
    Dispatch.register(_n)


class Execute(Enum):
    ALL = 0
    RANK_ZERO = 1


# ---------------------------------------------------------------------------------------------------- helpers
def _split_args_kwargs(chunks: int, *args, **kwargs):
    """Split every DataProto / DataProtoFuture argument into ``chunks`` parts (auto-padding when enabled)."""
    pad_size = None

    def split(x):
        nonlocal pad_size
        assert isinstance(x, (DataProto, DataProtoFuture)), f"expected DataProto, got {type(x)}"
        if isinstance(x, DataProto) and x.is_padding_enabled():
            x, ps = pad_dataproto_to_divisor(x, chunks)
            assert pad_size is None or pad_size == ps, "all padded arguments must need the same padding"
            pad_size = ps
        return x.chunk(chunks=chunks)

    s_args = [split(a) for a in args]
    s_kwargs = {k: split(v) for k, v in kwargs.items()}
    if pad_size is not None:
        s_kwargs["_pad_size"] = pad_size
    return s_args, s_kwargs


def dispatch_one_to_all(worker_group, *args, **kwargs):
    n = worker_group.world_size
    return tuple([a] * n for a in args), {k: [v] * n for k, v in kwargs.items()}


def dispatch_all_to_all(worker_group, *args, **kwargs):
    return args, kwargs


def collect_all_to_all(worker_group, output):
    return output


def dispatch_dp_compute(worker_group, *args, **kwargs):
    for a in list(args) + list(kwargs.values()):
        assert isinstance(a, (tuple, list)) and len(a) == worker_group.world_size
    return args, kwargs


def collect_dp_compute(worker_group, output):
    assert len(output) == worker_group.world_size
    return output


def _concat_data_proto_or_future(output: list):
    for o in output:
        assert type(o) is type(output[0])
    o = output[0]
    if isinstance(o, DataProto):
        return DataProto.concat(output)
    if isinstance(o, DataProtoFuture):
        return DataProtoFuture.concat(output)
    if hasattr(o, "result"):
        return DataProtoFuture.concat(output)
    raise NotImplementedError(f"cannot merge outputs of type {type(o)}")


def dispatch_dp_compute_data_proto(worker_group, *args, **kwargs):
    s_args, s_kwargs = _split_args_kwargs(worker_group.world_size, *args, **kwargs)
    return tuple(s_args), s_kwargs


def collect_dp_compute_data_proto(worker_group, output):
    for o in output:
        assert isinstance(o, (DataProto, DataProtoFuture)) or hasattr(o, "result"), f"expecting DataProto, got {type(o)}"
    return _concat_data_proto_or_future(collect_dp_compute(worker_group, output))


def dispatch_dp_compute_data_proto_with_func(worker_group, *args, **kwargs):
    assert callable(args[0]), "first argument must be a function"
    s_args, s_kwargs = _split_args_kwargs(worker_group.world_size, *args[1:], **kwargs)
    return tuple([[args[0]] * worker_group.world_size] + s_args), s_kwargs


def collect_dp_compute_metric(worker_group, output):
    return output


# ---------------------------------------------------------------------------------------------------- n-d mesh dispatch
def dispatch_nd_compute(dp_rank_mapping: list[int], dp_size: int, worker_group, *args, **kwargs):
    """Arguments are pre-split into ``dp_size`` chunks; worker i receives chunk ``dp_rank_mapping[i]`` (so tensor /
    sequence / pipeline peers of one data-parallel group all see the same chunk)."""
    def route(a):
        assert isinstance(a, (tuple, list)) and len(a) == dp_size
        return [a[dp_rank_mapping[i]] for i in range(worker_group.world_size)]

    return tuple(route(a) for a in args), {k: route(v) for k, v in kwargs.items()}


def collect_nd_compute(collect_mask: list[bool], worker_group, output):
    assert len(output) == worker_group.world_size
    return [output[i] for i in range(worker_group.world_size) if collect_mask[i]]


def dispatch_nd_compute_dataproto(dp_rank_mapping: list[int], dp_size: int, worker_group, *args, **kwargs):
    s_args, s_kwargs = _split_args_kwargs(dp_size, *args, **kwargs)
    pad = s_kwargs.pop("_pad_size", None)
    a, k = dispatch_nd_compute(dp_rank_mapping, dp_size, worker_group, *s_args, **s_kwargs)
    if pad is not None:
        k["_pad_size"] = pad
    return a, k


def collect_nd_compute_dataproto(collect_mask: list[bool], worker_group, output):
    output = collect_nd_compute(collect_mask, worker_group, output)
    return _concat_data_proto_or_future(output)


def make_nd_compute_dataproto_dispatch_fn(mesh_name: str) -> dict:
    """Dispatch by the data-parallel coordinate of mesh ``mesh_name`` that the workers registered at init time
    (``Worker._register_dispatch_collect_info``); results are collected from one rank per DP group."""
    def dispatch(worker_group, *args, **kwargs):
        info = worker_group.query_dispatch_info(mesh_name)
        dp_size = max(info) + 1
        return dispatch_nd_compute_dataproto(info, dp_size, worker_group, *args, **kwargs)

    def collect(worker_group, output):
        mask = worker_group.query_collect_info(mesh_name)
        return collect_nd_compute_dataproto(mask, worker_group, output)

    return {"dispatch_fn": dispatch, "collect_fn": collect}


# ---------------------------------------------------------------------------------------------------- registry
DISPATCH_MODE_FN_REGISTRY = {
    Dispatch.ONE_TO_ALL: {"dispatch_fn": dispatch_one_to_all, "collect_fn": collect_all_to_all},
    Dispatch.ALL_TO_ALL: {"dispatch_fn": dispatch_all_to_all, "collect_fn": collect_all_to_all},
    Dispatch.DP_COMPUTE: {"dispatch_fn": dispatch_dp_compute, "collect_fn": collect_dp_compute},
    Dispatch.DP_COMPUTE_PROTO: {"dispatch_fn": dispatch_dp_compute_data_proto, "collect_fn": collect_dp_compute_data_proto},
    Dispatch.DP_COMPUTE_PROTO_WITH_FUNC: {"dispatch_fn": dispatch_dp_compute_data_proto_with_func, "collect_fn": collect_dp_compute_data_proto},
    Dispatch.DP_COMPUTE_METRIC: {"dispatch_fn": dispatch_dp_compute_data_proto, "collect_fn": collect_dp_compute_metric},
    Dispatch.RANK_ZERO: {"dispatch_fn": dispatch_one_to_all, "collect_fn": lambda wg, out: out[0]},
    Dispatch.DIRECT_ROLLOUT_METHOD: {"dispatch_fn": dispatch_all_to_all, "collect_fn": collect_all_to_all},
}


def get_predefined_dispatch_fn(dispatch_mode):
    return DISPATCH_MODE_FN_REGISTRY[dispatch_mode]


def register_dispatch_mode(name: str, dispatch_fn: Callable, collect_fn: Callable):
    mode = Dispatch.register(name)
    DISPATCH_MODE_FN_REGISTRY[mode] = {"dispatch_fn": dispatch_fn, "collect_fn": collect_fn}
    return mode


def update_dispatch_mode(dispatch_mode, dispatch_fn: Callable, collect_fn: Callable):
    DISPATCH_MODE_FN_REGISTRY[dispatch_mode] = {"dispatch_fn": dispatch_fn, "collect_fn": collect_fn}


def get_predefined_execute_fn(execute_mode: Execute) -> dict:
    return {Execute.ALL: {"execute_fn_name": "execute_all"}, Execute.RANK_ZERO: {"execute_fn_name": "execute_rank_zero"}}[execute_mode]


def _check_dispatch_mode(mode):
    assert isinstance(mode, (Dispatch, dict)), f"dispatch_mode must be a Dispatch or a dict, got {type(mode)}"
    if isinstance(mode, dict):
        assert "dispatch_fn" in mode and "collect_fn" in mode


def _materialize_futures(*args, **kwargs):
    args = tuple(a.get() if isinstance(a, DataProtoFuture) else a for a in args)
    kwargs = {k: (v.get() if isinstance(v, DataProtoFuture) else v) for k, v in kwargs.items()}
    return args, kwargs


def register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.ALL, blocking: bool = True, materialize_futures: bool = True):
    """Mark a worker method as remotely callable through its worker group."""
    _check_dispatch_mode(dispatch_mode)
    assert isinstance(execute_mode, Execute)

    def decorator(func):
        if inspect.iscoroutinefunction(func):
            @wraps(func)
            async def inner(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                kwargs.pop("_pad_size", None)
                return await func(*args, **kwargs)
        else:
            @wraps(func)
            def inner(*args, **kwargs):
                if materialize_futures:
                    args, kwargs = _materialize_futures(*args, **kwargs)
                pad = kwargs.pop("_pad_size", None)
                out = func(*args, **kwargs)
                if pad and isinstance(out, DataProto):
                    out.meta_info["_pad_size"] = pad
                return out

        setattr(inner, MAGIC_ATTR, {"dispatch_mode": dispatch_mode, "execute_mode": execute_mode, "blocking": blocking})
        return inner

    return decorator
