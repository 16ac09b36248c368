"""Platform registry, device shims and NUMA pinning (against a fake NVML)."""

import os

import pytest

from verl_b200.plugin.platform import PlatformBase, PlatformCPU, PlatformCUDA, PlatformRegistry, get_platform, set_platform
from verl_b200.utils import device as dev
from verl_b200.utils import distributed as vd


def test_detection_registry_and_shims(monkeypatch):
    set_platform(None)
    p = get_platform()
    assert isinstance(p, PlatformCPU) and {"cuda", "cpu"} <= set(PlatformRegistry.registered_names())
    assert dev.get_device_name() == "cpu" and dev.get_nccl_backend() == "gloo" and dev.get_default_backend() == "gloo"
    assert not dev.is_support_ipc() and not dev.is_device_available() and dev.get_device_capability() == (None, None)
    assert dev.get_resource_name() == "CPU" and dev.get_visible_devices_keyword() == "CUDA_VISIBLE_DEVICES"
    c = PlatformCUDA()
    assert c.communication_backend_name() == "nccl" and c.process_group_backend() == "cpu:gloo,cuda:nccl" and c.is_ipc_supported()
    assert c.ray_resource_options(1) == {"num_gpus": 1} and c.get_device_capability() == (None, None) and not c.is_blackwell()
    with c.nvtx_range("x"):            # a no-op without a device
        pass
    monkeypatch.setenv("VERL_B200_PLATFORM", "nope")
    set_platform(None)
    with pytest.raises(ValueError, match="not registered"):
        get_platform()
    monkeypatch.delenv("VERL_B200_PLATFORM")
    set_platform(None)


def test_out_of_tree_platform_changes_every_shim(monkeypatch):
    @PlatformRegistry.register("fakechip")
    class Fake(PlatformCPU):
        device_name = "fakechip"
        vendor_name = "acme"

        def communication_backend_name(self):
            return "fccl"

        def ray_resource_name(self):
            return "FAKE"

        def visible_devices_envvar(self):
            return "FAKE_VISIBLE_DEVICES"

    with pytest.raises(TypeError):
        PlatformRegistry.register("bad")(dict)
    monkeypatch.setenv("VERL_B200_PLATFORM", "fakechip")
    set_platform(None)
    try:
        assert dev.get_device_name() == "fakechip" and dev.get_vendor() == "acme" and dev.get_nccl_backend() == "fccl"
        assert dev.get_visible_devices_keyword() == "FAKE_VISIBLE_DEVICES" and get_platform().ray_resource_options(2) == {"num_cpus": 2}
        cfg = {"trainer": {"device": "npu"}}
        dev.auto_set_device(cfg)
        assert cfg["trainer"]["device"] == "fakechip"
    finally:
        monkeypatch.delenv("VERL_B200_PLATFORM")
        set_platform(None)
    with pytest.raises(TypeError):
        set_platform(object())
    assert isinstance(get_platform(), PlatformBase)


class FakeNVML:
    """Two GPUs on two sockets of 8 CPUs each; records that only queries were made."""

    def __init__(self):
        self.calls = []

    def nvmlInit(self):
        self.calls.append("init")

    def nvmlShutdown(self):
        self.calls.append("shutdown")

    def nvmlDeviceGetHandleByIndex(self, i):
        self.calls.append(("index", i))
        if i > 1:
            raise RuntimeError("invalid index")
        return i

    def nvmlDeviceGetHandleByUUID(self, u):
        self.calls.append(("uuid", u))
        return {"GPU-aaa": 0, "GPU-bbb": 1}[u]

    def nvmlDeviceGetCpuAffinity(self, handle, words):
        self.calls.append(("affinity", handle))
        return [0xFF << (8 * handle)] + [0] * (words - 1)


def test_numa_affinity_pins_to_the_gpus_socket(monkeypatch):
    nv, pinned = FakeNVML(), []
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    assert vd.set_numa_affinity(1, nvml=nv, setter=pinned.append) == list(range(8, 16)) and pinned == [list(range(8, 16))]
    assert nv.calls == ["init", ("index", 1), ("affinity", 1), "shutdown"]          # queries only, library closed again
    # the visible-device list renumbers the devices; UUID entries are looked up as such
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "1,0")
    assert vd.set_numa_affinity(0, nvml=FakeNVML(), setter=pinned.append) == list(range(8, 16))
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "GPU-bbb")
    assert vd.cpus_near_device(0, FakeNVML()) == list(range(8, 16))
    # failures and the off switch leave the process alone
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "7")
    assert vd.set_numa_affinity(0, nvml=FakeNVML(), setter=pinned.append) is None
    monkeypatch.setenv("VERL_B200_NUMA_AFFINITY", "0")
    assert vd.set_numa_affinity(0, nvml=FakeNVML(), setter=pinned.append) is None and len(pinned) == 2
    monkeypatch.delenv("VERL_B200_NUMA_AFFINITY")
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES")
    # without an injected setter the mask is cut to the CPUs this process may use before sched_setaffinity is called
    before = os.sched_getaffinity(0)
    got = vd.set_numa_affinity(0, nvml=FakeNVML())
    assert (got is None or set(got) <= before) and os.sched_getaffinity(0) == (set(got) if got else before)
    os.sched_setaffinity(0, before)
