import signal
import subprocess
import sys
import os
import time

import pytest
import torch

from verl_b200.protocol import DataProto
from verl_b200.single_controller.base import ClassWithInitArgs, Dispatch, ResourcePool
from verl_b200.single_controller.base.decorator import MAGIC_ATTR, register, register_dispatch_mode
from verl_b200.single_controller.process import ProcessWorkerGroup, create_colocated_worker_cls
from verl_b200.single_controller.spmd import SPMDWorkerGroup

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _sc_workers import Adder, EchoWorker  # noqa: E402


@pytest.fixture(scope="module")
def wg():
    g = ProcessWorkerGroup(ResourcePool([4]), ClassWithInitArgs(EchoWorker, scale=1), name_prefix="t", use_gpu=False)
    yield g
    g.shutdown()


def test_env_contract(wg):
    envs = wg.env()
    assert [e["RANK"] for e in envs] == ["0", "1", "2", "3"] and all(e["WORLD_SIZE"] == "4" for e in envs)
    assert envs[0]["MASTER_ADDR"] == "127.0.0.1" and envs[0]["WG_PREFIX"] == "t" and len({e["MASTER_PORT"] for e in envs}) == 1


def test_dp_compute_proto_splits_and_concats(wg):
    out = wg.double(DataProto.from_dict(tensors={"x": torch.arange(8)}))
    assert out.batch["y"].tolist() == [0, 2, 4, 6, 8, 10, 12, 14] and out.batch["rank"].tolist() == [0, 0, 1, 1, 2, 2, 3, 3]


def test_auto_padding_roundtrip(wg):
    d = DataProto.from_dict(tensors={"x": torch.arange(6)}, auto_padding=True)
    out = wg.double(d)
    assert out.batch["y"].tolist() == [0, 2, 4, 6, 8, 10]


def test_nd_mesh_dispatch_replicates_within_group_and_collects_once(wg):
    out = wg.nd(DataProto.from_dict(tensors={"x": torch.arange(4)}))
    assert out.batch["x"].tolist() == [0, 1, 2, 3] and out.batch["rank"].tolist() == [0, 0, 2, 2]


def test_rank_zero_and_nonblocking(wg):
    assert wg.only_zero(5) == [(0, 5)]
    t0 = time.time()
    futs = wg.slow(0.3)
    assert time.time() - t0 < 0.25
    assert [f.result() for f in futs] == [0, 1, 2, 3]


def test_worker_exception_is_propagated(wg):
    with pytest.raises(RuntimeError, match="intentional failure"):
        wg.boom()
    assert wg.env()[0]["RANK"] == "0"     # the group survives a Python exception in a worker


def test_colocated_roles():
    cd = {"a": ClassWithInitArgs(Adder, 1), "b": ClassWithInitArgs(Adder, 10)}
    g = ProcessWorkerGroup(ResourcePool([2]), create_colocated_worker_cls(cd), use_gpu=False)
    try:
        views = g.spawn({"a", "b"})
        assert views["a"].add(1) == [2, 2] and views["b"].add(1) == [11, 11]
        assert g.a_add(5) == [6, 6]
    finally:
        g.shutdown()


def test_custom_dispatch_mode_and_magic_attr():
    mode = register_dispatch_mode("TEST_EVEN_ONLY", lambda wg, *a, **k: (a, k), lambda wg, out: out[::2])

    class W:
        @register(dispatch_mode=mode)
        def f(self):
            return 1

    assert getattr(W.f, MAGIC_ATTR)["dispatch_mode"] == mode and Dispatch.from_name("test_even_only") == mode
    with pytest.raises(ValueError):
        register_dispatch_mode("TEST_EVEN_ONLY", None, None)


def test_spmd_group_single_rank():
    g = SPMDWorkerGroup(cls_with_init_args=ClassWithInitArgs(EchoWorker, scale=3))
    out = g.double(DataProto.from_dict(tensors={"x": torch.arange(4)}))
    assert out.batch["y"].tolist() == [0, 6, 12, 18]


LIVENESS = r'''
import os, sys, time
sys.path.insert(0, os.environ["REPO"]); sys.path.insert(0, os.path.join(os.environ["REPO"], "tests"))
from verl_b200.single_controller.base import ClassWithInitArgs, ResourcePool
from verl_b200.single_controller.process import ProcessWorkerGroup
from _sc_workers import EchoWorker
if __name__ == "__main__":
    g = ProcessWorkerGroup(ResourcePool([2]), ClassWithInitArgs(EchoWorker), use_gpu=False)
    g.start_worker_aliveness_check(0.2)
    try:
        g.die()
    except Exception:
        pass
    time.sleep(30)
    print("controller survived", flush=True)
'''


def test_controller_aborts_when_a_worker_dies(tmp_path):
    """Host-side failure injection: a worker process exits; the watchdog raises SIGABRT in the controller."""
    script = tmp_path / "live.py"
    script.write_text(LIVENESS)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, str(script)], env=dict(os.environ, REPO=repo), capture_output=True, text=True, timeout=120)
    assert r.returncode == -signal.SIGABRT, (r.returncode, r.stdout[-500:], r.stderr[-500:])
    assert "controller survived" not in r.stdout


def test_resource_pools_split_merge_and_manager():
    from verl_b200.single_controller.base import ResourcePool, ResourcePoolManager, merge_resource_pool, split_resource_pool

    pool = ResourcePool([4, 4])
    a, b = split_resource_pool(pool, [6, 2])
    assert a.world_size == 6 and b.world_size == 2
    assert a.device_slots() == [(0, 0), (0, 1), (0, 2), (0, 3), (1, 0), (1, 1)] and b.device_slots() == [(1, 2), (1, 3)]
    assert b.local_rank_list() == [2, 3] and a.local_world_size_list() == [4, 4, 4, 4, 2, 2]
    halves = split_resource_pool(a, 3)                      # a slice can be split again
    assert [h.device_slots() for h in halves] == [[(0, 0), (0, 1), (0, 2)], [(0, 3), (1, 0), (1, 1)]]
    with pytest.raises(AssertionError):
        split_resource_pool(pool, 3)
    with pytest.raises(AssertionError):
        split_resource_pool(pool, [4, 3])
    m = merge_resource_pool(ResourcePool([2]), ResourcePool([4, 4]))
    assert m.store == [2, 4, 4] and m.world_size == 10
    with pytest.raises(AssertionError):
        merge_resource_pool(ResourcePool([2], max_colocate_count=1), ResourcePool([2], max_colocate_count=3))

    mgr = ResourcePoolManager({"train": [4], "rollout": [4]}, {"actor": "train", "critic": "train", "rollout": "rollout"}, available=8)
    pools = mgr.create_resource_pool()
    assert mgr.get_n_gpus() == 8 and mgr.get_resource_pool("critic") is pools["train"] and mgr.get_resource_pool("rollout").world_size == 4
    with pytest.raises(ValueError):
        ResourcePoolManager({"train": [8], "rollout": [4]}, {"actor": "train"}, available=8).create_resource_pool()


def test_worker_groups_on_sub_pools_get_their_slice_of_devices():
    """Two process worker groups on disjoint slices of one pool: LOCAL_RANK of every worker is its device index in the
    parent pool, ranks are numbered inside each group."""
    from tests._sc_workers import EnvWorker
    from verl_b200.single_controller.base import ClassWithInitArgs, ResourcePool, split_resource_pool
    from verl_b200.single_controller.process import ProcessWorkerGroup

    left, right = split_resource_pool(ResourcePool([3]), [1, 2])
    wg_l = ProcessWorkerGroup(left, ClassWithInitArgs(EnvWorker), use_gpu=False)
    wg_r = ProcessWorkerGroup(right, ClassWithInitArgs(EnvWorker), use_gpu=False)
    try:
        assert wg_l.env() == [("0", "1", "0")]
        assert wg_r.env() == [("0", "2", "1"), ("1", "2", "2")]
    finally:
        wg_l.shutdown()
        wg_r.shutdown()
