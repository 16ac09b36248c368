"""One fleet of rollout replicas per distillation teacher.

A teacher is a frozen model that only ever scores sequences, so it runs on rollout servers (``SamplingParams.prompt_logprobs``),
not on a training engine: ``num_replicas`` standalone server processes, each pinned to the devices it was given, behind one
load-balanced client. Several teachers (one per routing key, e.g. per data source) share the dedicated device list, which is cut
in the order the teachers are configured; a replica must not straddle two nodes unless it is at least a node wide.

Reference: ``verl/experimental/teacher_loop/teacher_model.py:38-228`` (replicas on a dedicated resource pool split per replica,
node-alignment check, per-teacher client).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

from verl_b200.workers.rollout.llm_server import LLMServerClient, LLMServerManager
from verl_b200.workers.rollout.replica import RolloutMode, RolloutReplica

__all__ = ["TeacherModelSpec", "TeacherModelManager", "build_teacher_fleet"]


@dataclass
class TeacherModelSpec:
    key: str
    model_path: str
    num_replicas: int = 1
    tensor_model_parallel_size: int = 1
    max_model_len: int = 4096
    max_num_seqs: int = 64
    gpu_memory_utilization: float = 0.85
    extra_args: list = field(default_factory=list)

    @property
    def per_replica_world_size(self) -> int:
        return int(self.tensor_model_parallel_size)

    @classmethod
    def from_config(cls, key: str, cfg) -> "TeacherModelSpec":
        g = (lambda k, d=None: cfg.get(k, d)) if hasattr(cfg, "get") else (lambda k, d=None: getattr(cfg, k, d))
        inf = g("inference", {}) or {}
        gi = (lambda k, d=None: inf.get(k, d)) if hasattr(inf, "get") else (lambda k, d=None: getattr(inf, k, d))
        path = g("model_path") or g("path") or g("preset")
        if not path:
            raise ValueError(f"teacher {key!r}: model_path is required")
        return cls(key=key, model_path=str(path), num_replicas=int(g("num_replicas", 1) or 1),
                   tensor_model_parallel_size=int(gi("tensor_model_parallel_size", 1) or 1), max_model_len=int(gi("max_model_len", 4096) or 4096),
                   max_num_seqs=int(gi("max_num_seqs", 64) or 64), gpu_memory_utilization=float(gi("gpu_memory_utilization", 0.85) or 0.85))


def check_node_alignment(key: str, start: int, num_replicas: int, width: int, gpus_per_node: int) -> None:
    """Replica i of a teacher takes devices [start + i*width, start + (i+1)*width) of the dedicated list. It must span exactly
    ``ceil(width / gpus_per_node)`` nodes — a linear cut that ignores node boundaries would otherwise put, say, a 4-GPU replica on
    the last GPU of one node and three of the next."""
    want = -(-width // gpus_per_node)
    for i in range(num_replicas):
        a = start + i * width
        span = (a + width - 1) // gpus_per_node - a // gpus_per_node + 1
        if span != want:
            raise ValueError(f"Teacher {key!r} replica {i} would take devices [{a}, {a + width}) and span {span} node(s); with "
                             f"{gpus_per_node} GPUs per node a replica of {width} should span {want}. Reorder the teachers or adjust "
                             "num_replicas / the inference parallelism so that every replica is aligned to node boundaries.")


class TeacherModelManager:
    """The replicas of ONE teacher and the client that balances over them. ``devices``: the device strings of this teacher's share
    (``num_replicas * per_replica_world_size`` of them; ``None`` entries let the server choose, which is what CPU tests use)."""

    def __init__(self, spec: TeacherModelSpec, devices: Sequence[Optional[str]], rollout_config=None, servers: Optional[dict] = None):
        self.spec = spec
        need = spec.num_replicas * spec.per_replica_world_size
        if servers is None and len(devices) != need:
            raise ValueError(f"Teacher {spec.key!r} expected {need} devices (num_replicas={spec.num_replicas} * per_replica_world_size="
                             f"{spec.per_replica_world_size}), but got {len(devices)}.")
        self.rollout_replicas: list = []
        if servers is not None:                      # servers that already exist (in-process engines, remote addresses)
            self._servers = dict(servers)
        else:
            if spec.per_replica_world_size != 1:
                raise NotImplementedError("teacher replicas score prompts on tensor_model_parallel_size=1 engines")
            extra = ["--max-num-seqs", str(spec.max_num_seqs), "--max-model-len", str(spec.max_model_len),
                     "--gpu-memory-utilization", str(spec.gpu_memory_utilization)] + list(spec.extra_args)
            suffix = spec.key.replace("/", "_")
            for i in range(spec.num_replicas):
                r = RolloutReplica(i, rollout_config or {}, mode=RolloutMode.STANDALONE).init_standalone(spec.model_path, device=devices[i], extra_args=extra)
                r.name = f"teacher_{suffix}_{i}"
                self.rollout_replicas.append(r)
            self._servers = {f"teacher_{suffix}_{i}": r.address for i, r in enumerate(self.rollout_replicas)}
        self.server_addresses = [v for v in self._servers.values() if isinstance(v, str)]
        self._client: Optional[LLMServerClient] = None

    def client(self) -> LLMServerClient:
        if self._client is None:
            self._client = LLMServerClient(self._servers)
        return self._client

    def prometheus_targets(self) -> list:
        return list(self.server_addresses)

    def shutdown(self) -> None:
        for r in self.rollout_replicas:
            r.shutdown()
        self.rollout_replicas = []


def build_teacher_fleet(teacher_models: dict, devices: Sequence[Optional[str]], gpus_per_node: int = 8, rollout_config=None) -> dict:
    """``{key: TeacherModelManager}`` for ``distillation.teacher_models``, cutting ``devices`` in configuration order."""
    specs = [TeacherModelSpec.from_config(k, v) for k, v in teacher_models.items()]
    total = sum(s.num_replicas * s.per_replica_world_size for s in specs)
    if total != len(devices):
        raise ValueError(f"the teachers need {total} devices, the dedicated pool has {len(devices)}")
    out, start = {}, 0
    for s in specs:
        n = s.num_replicas * s.per_replica_world_size
        if all(d is not None for d in devices[start:start + n]):
            check_node_alignment(s.key, start, s.num_replicas, s.per_replica_world_size, gpus_per_node)
        out[s.key] = TeacherModelManager(s, list(devices[start:start + n]), rollout_config)
        start += n
    return out
