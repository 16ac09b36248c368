"""PRIME-style reward manager: every sample of the batch is scored in a pool of worker processes with a per-sample time
limit, so that one pathological completion (an endless loop inside a code or symbolic-math checker) costs its own time-out
and a zero score instead of stalling the step. The pool's processes are terminated after every batch, which also reaps
checkers that ignored the time-out. Scores are written at the last valid response token and kept as ``acc`` in the batch.

Reference: ``verl/workers/reward_manager/prime.py`` (process-pool scoring :30-103, manager :106-189).
"""

from __future__ import annotations

import asyncio
from concurrent.futures import ProcessPoolExecutor
from functools import partial

import torch

from verl_b200.protocol import DataProto
from verl_b200.utils.reward_score import default_compute_score

from .registry import register

__all__ = ["PrimeRewardManager", "run_reward_scoring"]


async def _score_one(fn, completion, reference, task, extra, pool, timeout: float):
    loop = asyncio.get_running_loop()
    try:
        return await asyncio.wait_for(loop.run_in_executor(pool, partial(fn, task, completion, reference, extra)), timeout=timeout)
    except asyncio.TimeoutError:
        print(f"[Timeout] reward scoring timed out: {str(completion)[:80]}")
    except Exception as e:  # noqa: BLE001
        print(f"[Error] reward scoring failed: {e}; completion: {str(completion)[:80]}")
    return None


def _as_float(r) -> float:
    if r is None or isinstance(r, Exception):
        return 0.0
    if isinstance(r, (int, float, bool)):
        return float(r)
    if isinstance(r, dict):
        return float(r.get("score", 0.0))
    return float(r[0])


def run_reward_scoring(fn, completions, references, tasks, extra_info=None, num_processes: int = 64, timeout: float = 300.0) -> list:
    """``fn(task, completion, reference, extra)`` for every sample, in ``num_processes`` workers; failures and time-outs score 0."""
    extra_info = list(extra_info) if extra_info is not None else [None] * len(tasks)

    async def run():
        pool = ProcessPoolExecutor(max_workers=max(1, min(num_processes, len(tasks) or 1)))
        try:
            return await asyncio.gather(*[_score_one(fn, c, r, t, e, pool, timeout) for c, r, t, e in zip(completions, references, tasks, extra_info)])
        finally:
            procs = list(getattr(pool, "_processes", {}).values())
            pool.shutdown(wait=False, cancel_futures=True)
            for p in procs:                       # a checker stuck in native code does not see the cancellation
                try:
                    p.terminate()
                    p.join(timeout=5)
                    if p.is_alive():
                        p.kill()
                except Exception:  # noqa: BLE001
                    pass

    loop = asyncio.new_event_loop()
    try:
        return [_as_float(r) for r in loop.run_until_complete(run())]
    finally:
        loop.close()


@register("prime")
class PrimeRewardManager:
    def __init__(self, tokenizer=None, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source", num_processes: int = 64,
                 timeout: float = 300.0, **kwargs):
        self.tokenizer = tokenizer
        self.num_examine = num_examine
        self.compute_score = compute_score or default_compute_score
        self.reward_fn_key = reward_fn_key
        self.num_processes, self.timeout = num_processes, timeout

    def _decode(self, ids) -> str:
        if self.tokenizer is not None:
            return self.tokenizer.decode(ids, skip_special_tokens=True)
        return " ".join(str(int(t)) for t in ids)

    def verify(self, data: DataProto) -> list:
        """Score the whole batch; the scores also land in ``data.batch["acc"]``."""
        P = data.batch["prompts"].shape[-1]
        n_resp = data.batch["attention_mask"][:, P:].sum(-1)
        texts = [self._decode(data.batch["responses"][i, :int(n_resp[i])]) for i in range(len(data))]
        rm = data.non_tensor_batch.get("reward_model")
        truths = [(rm[i] or {}).get("ground_truth") if rm is not None else None for i in range(len(data))]
        tasks = list(data.non_tensor_batch[self.reward_fn_key])
        extra = data.non_tensor_batch.get("extra_info")
        try:
            scores = run_reward_scoring(self.compute_score, texts, truths, tasks, extra, self.num_processes, self.timeout)
        except Exception as e:  # noqa: BLE001
            print(f"[Error] unexpected failure during reward scoring, all samples score 0: {e}")
            scores = [0.0] * len(texts)
        data.batch["acc"] = torch.tensor(scores, dtype=torch.float32)
        return scores

    def __call__(self, data: DataProto, return_dict: bool = False):
        if "rm_scores" in data.batch.keys():
            return {"reward_tensor": data.batch["rm_scores"], "reward_extra_info": {}} if return_dict else data.batch["rm_scores"]
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        P = data.batch["prompts"].shape[-1]
        n_resp = data.batch["attention_mask"][:, P:].sum(-1)
        scores = self.verify(data)
        shown: dict = {}
        for i, s in enumerate(scores):
            if int(n_resp[i]) > 0:
                reward[i, int(n_resp[i]) - 1] = s
            src = data.non_tensor_batch[self.reward_fn_key][i]
            if shown.get(src, 0) < self.num_examine:
                shown[src] = shown.get(src, 0) + 1
                print("[response]", self._decode(data.batch["responses"][i, :int(n_resp[i])]), "\n[score]", s)
        return {"reward_tensor": reward, "reward_extra_info": {"acc": scores}} if return_dict else reward
