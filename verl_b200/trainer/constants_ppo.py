"""Environment that a training job's processes start with.

`WORKER_ENV_DEFAULTS` are defaults, not overrides: `get_worker_runtime_env` leaves out every variable the launching shell already set, so
a user's ``NCCL_DEBUG=INFO`` survives.  ``run_ppo`` applies the result to its own process before any worker or process group exists; torchrun ranks run it
themselves and spawned workers inherit it.  Config-dependent entries (optional keys: add them with ``+trainer.disable_nvls=true`` and the like):

* ``trainer.runtime_env.env_vars`` — free-form additions from the config, applied last among the defaults;
* a run profiled with the torch profiler (``global_profiler.tool=torch``) disables NVTX injection, which otherwise doubles every range;
* ``trainer.disable_nvls=true`` turns NCCL's in-switch reduction off (``NCCL_NVLS_ENABLE=0``) for jobs whose ranks may leave between
  steps: a rank that dies while bound to a multicast object can fault its peers.

Reference: ``verl/trainer/constants_ppo.py:64-152`` (``PPO_RAY_RUNTIME_ENV``, ``get_ppo_ray_runtime_env``).
"""
from __future__ import annotations

import os
from typing import Mapping, Optional

NVTX_INJECTION_ENV = "NVTX_INJECTION64_PATH"
_NVTX_INJECTION_DISABLED = "/nonexistent/disabled-nvtx-injection.so"

WORKER_ENV_DEFAULTS = {
    "TOKENIZERS_PARALLELISM": "true",      # tokenisation happens before workers fork their own threads
    "NCCL_DEBUG": "WARN",
    "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1",   # a failed collective raises on the host instead of hanging the step
    "CUDA_MODULE_LOADING": "LAZY",
}


def _select(config, dotted: str, default=None):
    cur = config
    for part in dotted.split("."):
        if not isinstance(cur, Mapping) or part not in cur:
            return default
        cur = cur[part]
    return default if cur is None else cur


def get_worker_runtime_env(config=None, environ: Optional[Mapping[str, str]] = None) -> dict:
    """``{"env_vars": {...}}`` with the defaults the current environment does not already decide."""
    environ = os.environ if environ is None else environ
    wanted = dict(WORKER_ENV_DEFAULTS)
    if config is not None:
        if _select(config, "global_profiler.tool") == "torch":
            wanted[NVTX_INJECTION_ENV] = _NVTX_INJECTION_DISABLED
        if bool(_select(config, "trainer.disable_nvls", False)):
            wanted["NCCL_NVLS_ENABLE"] = "0"
        wanted.update({str(k): str(v) for k, v in (_select(config, "trainer.runtime_env.env_vars", {}) or {}).items()})
    return {"env_vars": {k: v for k, v in wanted.items() if k not in environ}}


def apply_worker_runtime_env(config=None) -> dict:
    """Sets the missing variables in this process (child processes inherit them); returns what was set."""
    env = get_worker_runtime_env(config)["env_vars"]
    os.environ.update(env)
    return env


# name under which recipes written against the reference import it
get_ppo_ray_runtime_env = get_worker_runtime_env
