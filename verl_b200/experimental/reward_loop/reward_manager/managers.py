"""Per-sample reward managers of the reward loop (reference: ``verl/experimental/reward_loop/reward_manager/{naive,dapo,
gdpo,limited,remote}.py``). All return ``{"reward_score": float, "reward_extra_info": dict}`` from ``run_single``."""

from __future__ import annotations

import asyncio
import inspect
import time
from typing import Callable, Optional

from verl_b200.utils.reward_score import default_compute_score

from ..reward_loop import register_reward_loop

__all__ = ["RewardLoopManagerBase", "NaiveRewardLoopManager", "DAPORewardLoopManager", "GDPORewardLoopManager", "RateLimitedRewardLoopManager",
           "RemoteRewardLoopManager"]


def _cfg(cfg, path, default=None):
    cur = cfg
    for p in path.split("."):
        if cur is None:
            return default
        cur = cur.get(p, None) if hasattr(cur, "get") else getattr(cur, p, None)
    return default if cur is None else cur


class RewardLoopManagerBase:
    def __init__(self, config, tokenizer, compute_score: Optional[Callable] = None, rm_client=None, **kwargs):
        self.config, self.tokenizer, self.rm_client = config, tokenizer, rm_client
        self.compute_score = compute_score or default_compute_score
        self._is_async = inspect.iscoroutinefunction(self.compute_score)

    def _text(self, sample: dict) -> str:
        if "response_str" in sample:
            return sample["response_str"]
        return self.tokenizer.decode(sample["response_ids"], skip_special_tokens=True)

    async def _score(self, sample: dict, text: str):
        rm = sample.get("reward_model") or {}
        kw = dict(data_source=sample.get("data_source"), solution_str=text, ground_truth=rm.get("ground_truth") if hasattr(rm, "get") else None,
                  extra_info=sample.get("extra_info"))
        if self._is_async:
            return await self.compute_score(**kw)
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.compute_score(**kw))

    @staticmethod
    def _unpack(res) -> tuple[float, dict]:
        if isinstance(res, dict):
            return float(res["score"]), {k: v for k, v in res.items()}
        return float(res), {"acc": float(res)}

    async def run_single(self, sample: dict) -> dict:
        raise NotImplementedError


@register_reward_loop("naive")
class NaiveRewardLoopManager(RewardLoopManagerBase):
    async def run_single(self, sample: dict) -> dict:
        score, info = self._unpack(await self._score(sample, self._text(sample)))
        return {"reward_score": score, "reward_extra_info": info}


@register_reward_loop("dapo")
class DAPORewardLoopManager(RewardLoopManagerBase):
    """Adds DAPO's soft over-length penalty: linear from 0 to −penalty_factor over the last ``overlong_buffer.len`` tokens."""

    async def run_single(self, sample: dict) -> dict:
        score, info = self._unpack(await self._score(sample, self._text(sample)))
        ob = _cfg(self.config, "reward.reward_kwargs.overlong_buffer_cfg", None) or _cfg(self.config, "reward_model.overlong_buffer", None)
        if ob and ob.get("enable", False):
            max_len = int(_cfg(self.config, "reward.reward_kwargs.max_resp_len", None) or _cfg(self.config, "data.max_response_length"))
            buf = int(ob["len"])
            exceed = sample["valid_response_length"] - (max_len - buf)
            pen = min(-exceed / buf * float(ob["penalty_factor"]), 0.0)
            score += pen
            if ob.get("log", False):
                info["overlong_reward"], info["overlong"] = pen, pen < 0
        return {"reward_score": score, "reward_extra_info": info}


@register_reward_loop("gdpo")
class GDPORewardLoopManager(RewardLoopManagerBase):
    """Multi-component rewards for GDPO: the scorer returns a dict of named components; each is kept in the extra info
    (``reward_components``) so the estimator can normalise them per group before summing; the scalar is their sum."""

    async def run_single(self, sample: dict) -> dict:
        res = await self._score(sample, self._text(sample))
        if isinstance(res, dict) and "components" in res:
            comps = {k: float(v) for k, v in res["components"].items()}
            return {"reward_score": float(sum(comps.values())), "reward_extra_info": {"reward_components": comps, **{f"reward/{k}": v for k, v in comps.items()}}}
        score, info = self._unpack(res)
        return {"reward_score": score, "reward_extra_info": {"reward_components": {"score": score}, **info}}


class _TokenBucket:
    def __init__(self, rate_per_s: float, burst: int):
        self.rate, self.cap = float(rate_per_s), float(burst)
        self.tokens, self.t = float(burst), time.monotonic()
        self.lock = asyncio.Lock()

    async def take(self):
        while True:
            async with self.lock:
                now = time.monotonic()
                self.tokens = min(self.cap, self.tokens + (now - self.t) * self.rate)
                self.t = now
                if self.tokens >= 1:
                    self.tokens -= 1
                    return
                wait = (1 - self.tokens) / self.rate
            await asyncio.sleep(wait)


@register_reward_loop("limited")
class RateLimitedRewardLoopManager(NaiveRewardLoopManager):
    """For scorers that call metered services: at most ``max_concurrent`` calls in flight and ``max_rpm`` per minute
    (token bucket), with a per-call timeout after which the sample scores 0."""

    _buckets: dict = {}

    def __init__(self, config, tokenizer, compute_score=None, rm_client=None, **kwargs):
        super().__init__(config, tokenizer, compute_score, rm_client)
        rk = _cfg(config, "reward.reward_kwargs", {}) or {}
        self.max_concurrent = int(rk.get("max_concurrent", 8))
        self.max_rpm = float(rk.get("max_rpm", 0) or 0)
        self.timeout_s = float(rk.get("timeout", 300))
        self._sem: Optional[asyncio.Semaphore] = None
        self._bucket: Optional[_TokenBucket] = None

    async def run_single(self, sample: dict) -> dict:
        if self._sem is None:
            self._sem = asyncio.Semaphore(self.max_concurrent)
            self._bucket = _TokenBucket(self.max_rpm / 60.0, max(1, int(self.max_rpm / 60.0) or 1)) if self.max_rpm > 0 else None
        async with self._sem:
            if self._bucket is not None:
                await self._bucket.take()
            try:
                return await asyncio.wait_for(super().run_single(sample), self.timeout_s)
            except asyncio.TimeoutError:
                return {"reward_score": 0.0, "reward_extra_info": {"acc": 0.0, "timeout": True}}


@register_reward_loop("remote")
class RemoteRewardLoopManager(RewardLoopManagerBase):
    """Scores with a reward MODEL behind a server: ``rm_client`` is an ``LLMServerClient``-like object. Discriminative
    models are queried with the prompt+response tokens and the scalar comes back in ``extra_fields["score"]``;
    generative judges return text that ``compute_score`` (or the default ``"Score: x"`` parser) turns into a number."""

    async def run_single(self, sample: dict) -> dict:
        from verl_b200.workers.rollout.engine import SamplingParams

        if self.rm_client is None:
            raise RuntimeError("the remote reward manager needs an rm_client")
        ids = list(sample.get("prompt_ids", [])) + list(sample["response_ids"])
        out = await self.rm_client.generate(None, ids, SamplingParams(temperature=0.0, max_tokens=int(_cfg(self.config, "reward.reward_kwargs.judge_max_tokens", 1))))
        if "score" in (out.extra_fields or {}):
            score = float(out.extra_fields["score"])
        else:
            import re

            text = self.tokenizer.decode(out.token_ids, skip_special_tokens=True)
            m = re.findall(r"[-+]?\d*\.?\d+", text)
            score = float(m[-1]) if m else 0.0
        return {"reward_score": score, "reward_extra_info": {"rm_score": score}}
