"""Rollout replicas: one serving instance of the inference engine plus how it relates to the trainer.

* ``HYBRID``      the replica lives in the trainer's process and reads the trainer's resident weights (zero-copy sync);
* ``COLOCATED``   same GPU, own copy of the weights, refreshed through a checkpoint-engine backend;
* ``STANDALONE``  own process / GPU, reached over HTTP (``python -m verl_b200.workers.rollout.replica``).

Reference: ``verl/workers/rollout/replica.py:49-390`` (RolloutMode, RolloutReplica, registry of vllm/sglang/trtllm
replicas). Here there is one engine, so the registry maps every reference name onto it.
"""

from __future__ import annotations

import enum
import os
import subprocess
import sys
import time
from typing import Optional

__all__ = ["RolloutMode", "RolloutReplica", "get_rollout_replica_class", "ROLLOUT_REPLICA_REGISTRY"]


class RolloutMode(enum.Enum):
    HYBRID = "hybrid"
    COLOCATED = "colocated"
    STANDALONE = "standalone"


class RolloutReplica:
    def __init__(self, replica_rank: int, config, model_config=None, mode: RolloutMode = RolloutMode.HYBRID):
        self.replica_rank, self.config, self.model_config, self.mode = replica_rank, config, model_config, mode
        self.server = None            # AsyncRolloutServer (in-process modes)
        self.address: Optional[str] = None
        self._stop_http = None
        self._proc: Optional[subprocess.Popen] = None

    # ------------------------------------------------------------------ launch
    def init_hybrid(self, engine, eos_token_id=None, tokenizer=None, http: bool = False):
        """Wrap an engine that already exists in this process (built by the actor/rollout worker)."""
        from verl_b200.workers.rollout.async_server import AsyncRolloutServer, serve_http

        self.server = AsyncRolloutServer(engine, eos_token_id=eos_token_id, tokenizer=tokenizer, name=f"replica-{self.replica_rank}")
        if http:
            self.address, self._stop_http = serve_http(self.server)
        return self

    def init_standalone(self, model: str, port: int = 0, device: Optional[str] = None, extra_args=(), timeout: float = 300.0):
        """Start ``python -m verl_b200.workers.rollout.replica`` as a child process and wait for its address file."""
        import tempfile

        addr_file = tempfile.mktemp(prefix="verl_b200_replica_")
        env = dict(os.environ)
        cmd = [sys.executable, "-m", "verl_b200.workers.rollout.replica", "--model", model, "--port", str(port), "--address-file", addr_file,
               "--name", f"replica-{self.replica_rank}", "--parent-pid", str(os.getpid()), *extra_args]
        if device is not None:
            # the other GPUs stay visible: weight hand-off maps the trainer's export buffer through CUDA IPC
            cmd += ["--device", str(device)]
        self._proc = subprocess.Popen(cmd, env=env)
        t0 = time.time()
        while not os.path.exists(addr_file):
            if self._proc.poll() is not None:
                raise RuntimeError(f"standalone replica exited with code {self._proc.returncode}")
            if time.time() - t0 > timeout:
                self._proc.kill()
                raise TimeoutError("standalone replica did not come up")
            time.sleep(0.1)
        self.address = open(addr_file).read().strip()
        os.unlink(addr_file)
        self.mode = RolloutMode.STANDALONE
        return self

    def init_remote(self, address: str):
        """Attach to a replica that already serves at ``host:port`` (started by another job or by ``init_standalone``)."""
        self.address, self.mode = address, RolloutMode.STANDALONE
        return self

    # ------------------------------------------------------------------ control
    def _post(self, path: str, body: Optional[dict] = None, timeout: float = 600.0) -> dict:
        import json
        import urllib.request

        req = urllib.request.Request(f"http://{self.address}{path}", data=json.dumps(body or {}).encode(), headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return json.loads(r.read().decode())

    def _get(self, path: str, timeout: float = 600.0) -> dict:
        import json
        import urllib.request

        with urllib.request.urlopen(f"http://{self.address}{path}", timeout=timeout) as r:
            return json.loads(r.read().decode())

    def wake_up(self):
        if self.server is not None:
            self.server.wake_up()
        elif self.address:
            self._post("/wake_up")

    def sleep(self):
        if self.server is not None:
            self.server.sleep()
        elif self.address:
            self._post("/sleep")

    def abort_all_requests(self):
        if self.server is not None:
            self.server.abort_all_requests()
        elif self.address:
            self._post("/abort")

    def update_weights(self, source: dict) -> int:
        """Hand new weights to the replica (see ``AsyncRolloutServer.update_weights``); returns its weights version."""
        if self.server is not None:
            return self.server.update_weights(source)
        return int(self._post("/update_weights", source)["weights_version"])

    def weights_version(self, checksum: bool = False) -> dict:
        if self.server is not None:
            d = {"weights_version": getattr(self.server, "weights_version", 0)}
            if checksum:
                d["checksum"] = self.server.weights_checksum()
            return d
        return self._get("/weights_version" + ("?checksum=1" if checksum else ""))

    def shutdown(self):
        if self._stop_http:
            self._stop_http()
        if self.server is not None:
            self.server.shutdown()
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=20)
            except subprocess.TimeoutExpired:
                self._proc.kill()


ROLLOUT_REPLICA_REGISTRY = {name: RolloutReplica for name in ("native", "vllm", "sglang", "trtllm", "hf")}


def get_rollout_replica_class(name: str):
    """Every engine name of the reference's configs resolves to the in-house replica."""
    if name not in ROLLOUT_REPLICA_REGISTRY:
        raise ValueError(f"unknown rollout engine {name!r}; known: {sorted(ROLLOUT_REPLICA_REGISTRY)}")
    return ROLLOUT_REPLICA_REGISTRY[name]


def main(argv=None):
    """Standalone replica process: build the model (preset name or HF directory), serve HTTP until terminated."""
    import argparse
    import signal

    import torch

    from verl_b200.models.config import PRESETS, ModelConfig
    from verl_b200.models.transformer import DecoderLM
    from verl_b200.workers.rollout.async_server import AsyncRolloutServer, serve_http
    from verl_b200.workers.rollout.engine import InferenceEngine

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--address-file", default=None)
    ap.add_argument("--name", default="replica-0")
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-model-len", type=int, default=2048)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.8)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", type=int, default=0, help="CUDA device index of this replica")
    ap.add_argument("--parent-pid", type=int, default=0, help="exit when this process is gone (a replica must not outlive the job that started it)")
    a = ap.parse_args(argv)
    dev = "cpu"
    if torch.cuda.is_available():
        torch.cuda.set_device(a.device)
        dev = f"cuda:{a.device}"
    tok = None
    if a.model in PRESETS:
        cfg = PRESETS[a.model]
        model = DecoderLM(cfg, dtype=torch.bfloat16 if dev != "cpu" else torch.float32, device=dev, seed=a.seed)
    else:
        from verl_b200.models.hf_io import load_hf_weights

        cfg = ModelConfig.from_pretrained(a.model)
        model = DecoderLM(cfg, dtype=torch.bfloat16 if dev != "cpu" else torch.float32, device=dev, init=False)
        load_hf_weights(model, a.model)
        try:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(a.model)
        except Exception:  # noqa: BLE001 - token-id endpoints still work
            tok = None
    eng = InferenceEngine(model, max_num_seqs=a.max_num_seqs, max_model_len=a.max_model_len, num_blocks=a.num_blocks,
                          gpu_memory_utilization=a.gpu_memory_utilization)
    server = AsyncRolloutServer(eng, eos_token_id=cfg.eos_token_id, tokenizer=tok, name=a.name)
    addr, stop = serve_http(server, a.host, a.port)
    if a.address_file:
        with open(a.address_file + ".tmp", "w") as f:
            f.write(addr)
        os.replace(a.address_file + ".tmp", a.address_file)
    print(f"[{a.name}] serving on {addr}", flush=True)
    done = [False]
    signal.signal(signal.SIGTERM, lambda *_: done.__setitem__(0, True))
    try:
        while not done[0]:
            time.sleep(0.2)
            if a.parent_pid and os.getppid() != a.parent_pid:
                break
    except KeyboardInterrupt:
        pass
    stop()
    server.shutdown()


if __name__ == "__main__":
    main()
