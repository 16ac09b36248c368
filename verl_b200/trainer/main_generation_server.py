"""Batch generation through standalone rollout servers and their OpenAI-style chat endpoint:

    python -m verl_b200.trainer.main_generation_server model.path=<hf dir or preset> data.path=prompts.parquet \\
        data.output_path=gen.parquet data.n_samples=4 rollout.num_replicas=2 rollout.temperature=1.0 rollout.response_length=512

Replicas are started as child processes (one per visible GPU, or on CPU), prompts (chat message lists under
``data.prompt_key``) are spread over them with bounded concurrency, and the input table is written back with a
``responses`` column (reference: ``verl/trainer/main_generation_server.py:40-150``).
"""

from __future__ import annotations

import asyncio
import copy
import sys

from verl_b200.utils.config import Config, apply_overrides

DEFAULT = {"model": {"path": None}, "data": {"path": None, "output_path": "generations.parquet", "prompt_key": "prompt", "n_samples": 1,
                                             "max_concurrency": 256},
           "rollout": {"num_replicas": 1, "temperature": 1.0, "top_p": 1.0, "top_k": -1, "response_length": 512, "max_model_len": 4096,
                       "gpu_memory_utilization": 0.8, "addresses": None}}


async def _generate_all(addresses, prompts, cfg):
    import aiohttp

    sem = asyncio.Semaphore(int(cfg.data.max_concurrency))
    ro = cfg.rollout

    async def one(session, i, messages):
        async with sem:
            body = {"model": cfg.model.path, "messages": list(messages), "n": int(cfg.data.n_samples), "temperature": float(ro.temperature),
                    "top_p": float(ro.top_p), "top_k": int(ro.top_k), "max_tokens": int(ro.response_length)}
            async with session.post(f"http://{addresses[i % len(addresses)]}/v1/chat/completions", json=body) as resp:
                resp.raise_for_status()
                d = await resp.json()
            return [c["message"]["content"] for c in d["choices"]]

    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None)) as session:
        return await asyncio.gather(*[one(session, i, m) for i, m in enumerate(prompts)])


def main(argv=None):
    import pandas as pd

    from verl_b200.workers.rollout.replica import RolloutReplica

    data = copy.deepcopy(DEFAULT)
    apply_overrides(data, list(sys.argv[1:] if argv is None else argv))
    cfg = Config(data)
    df = pd.read_parquet(cfg.data.path)
    prompts = [list(p) for p in df[cfg.data.prompt_key]]
    replicas = []
    addresses = list(cfg.rollout.addresses) if cfg.rollout.get("addresses") else None
    try:
        if addresses is None:
            import torch

            ngpu = torch.cuda.device_count()
            for r in range(int(cfg.rollout.num_replicas)):
                rep = RolloutReplica(r, cfg.rollout).init_standalone(
                    cfg.model.path, device=str(r % ngpu) if ngpu else None,
                    extra_args=["--max-model-len", str(cfg.rollout.max_model_len), "--gpu-memory-utilization", str(cfg.rollout.gpu_memory_utilization)])
                replicas.append(rep)
            addresses = [r.address for r in replicas]
        df["responses"] = asyncio.run(_generate_all(addresses, prompts, cfg))
    finally:
        for r in replicas:
            r.shutdown()
    df.to_parquet(cfg.data.output_path)
    print(f"wrote {len(df)} rows x {cfg.data.n_samples} samples to {cfg.data.output_path}")
    return df


if __name__ == "__main__":
    main()
