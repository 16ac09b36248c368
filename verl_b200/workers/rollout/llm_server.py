"""Client side of the rollout servers: load balancing across replicas, sticky sessions, abort/resume, fleet manager.

Reference: ``verl/workers/rollout/llm_server.py:43-364`` (``LLMServerManager``, ``LLMServerClient``,
``FullyAsyncLLMServerClient``) and ``router.py:32-397`` (``GlobalRequestLoadBalancer``).
"""

from __future__ import annotations

import asyncio
import hashlib
import uuid
from collections import OrderedDict
from typing import Optional, Sequence

from verl_b200.workers.rollout.engine import SamplingParams, TokenOutput

__all__ = ["GlobalRequestLoadBalancer", "LLMServerClient", "FullyAsyncLLMServerClient", "LLMServerManager"]


class GlobalRequestLoadBalancer:
    """Sticky-session routing with a bounded LRU map; new sessions go to the server with the fewest requests in flight
    (ties broken by a deterministic hash of the request id, so concurrent clients spread evenly)."""

    def __init__(self, server_ids: Sequence[str], max_cache_size: int = 10000):
        self.servers: list[str] = list(server_ids)
        self.inflight: dict[str, int] = {s: 0 for s in self.servers}
        self.sticky: "OrderedDict[str, str]" = OrderedDict()
        self.max_cache_size = max_cache_size

    def add_server(self, sid: str):
        if sid not in self.inflight:
            self.servers.append(sid)
            self.inflight[sid] = 0

    def remove_server(self, sid: str):
        if sid in self.inflight:
            self.servers.remove(sid)
            del self.inflight[sid]
            for k in [k for k, v in self.sticky.items() if v == sid]:
                del self.sticky[k]

    def acquire(self, request_id: str) -> str:
        if not self.servers:
            raise RuntimeError("no rollout servers registered")
        sid = self.sticky.get(request_id)
        if sid is None or sid not in self.inflight:
            low = min(self.inflight.values())
            cands = [s for s in self.servers if self.inflight[s] == low]
            h = int(hashlib.md5(request_id.encode()).hexdigest(), 16)
            sid = cands[h % len(cands)]
            self.sticky[request_id] = sid
            if len(self.sticky) > self.max_cache_size:
                self.sticky.popitem(last=False)
        else:
            self.sticky.move_to_end(request_id)
        self.inflight[sid] += 1
        return sid

    def release(self, sid: str):
        if sid in self.inflight:
            self.inflight[sid] = max(0, self.inflight[sid] - 1)


class LLMServerClient:
    """``await client.generate(request_id, prompt_ids, sampling_params)`` → ``TokenOutput``.

    ``servers`` maps a server id to either an in-process ``AsyncRolloutServer`` or an ``"host:port"`` address.
    """

    def __init__(self, servers: dict, balancer: Optional[GlobalRequestLoadBalancer] = None):
        self.servers = dict(servers)
        self.balancer = balancer or GlobalRequestLoadBalancer(list(self.servers))
        self._session = None
        self.closed = False     # set at shutdown: aborted requests are then returned as they are instead of being resumed

    async def _http(self):
        import aiohttp

        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None))
        return self._session

    async def _call(self, target, prompt_ids, sp: SamplingParams, request_id: str, multi_modal=None) -> TokenOutput:
        if isinstance(target, str):
            if multi_modal:
                raise NotImplementedError("image inputs are only passed to in-process servers (the HTTP protocol carries token ids)")
            sess = await self._http()
            body = {"prompt_ids": list(prompt_ids), "request_id": request_id,
                    "sampling_params": {"temperature": sp.temperature, "top_p": sp.top_p, "top_k": sp.top_k, "max_tokens": sp.max_tokens,
                                        "ignore_eos": sp.ignore_eos, "seed": sp.seed, "stop_token_ids": list(sp.stop_token_ids),
                                        "prompt_logprobs": sp.prompt_logprobs if sp.prompt_logprobs >= 0 else None}}
            async with sess.post(f"http://{target}/generate", json=body) as resp:
                resp.raise_for_status()
                d = await resp.json()
            return TokenOutput(token_ids=d["token_ids"], log_probs=d.get("log_probs"), stop_reason=d.get("stop_reason"),
                               num_preempted=d.get("num_preempted", 0), extra_fields=d.get("extra_fields") or {})
        return await (target.generate(prompt_ids, sp, request_id, multi_modal) if multi_modal else target.generate(prompt_ids, sp, request_id))

    async def generate(self, request_id: Optional[str], prompt_ids, sampling_params: Optional[SamplingParams] = None,
                       multi_modal: Optional[dict] = None) -> TokenOutput:
        request_id = request_id or uuid.uuid4().hex
        sp = sampling_params or SamplingParams()
        sid = self.balancer.acquire(request_id)
        try:
            return await self._call(self.servers[sid], prompt_ids, sp, request_id, multi_modal)
        finally:
            self.balancer.release(sid)

    async def close(self):
        if self._session is not None and not self._session.closed:
            await self._session.close()


class FullyAsyncLLMServerClient(LLMServerClient):
    """Survives aborts (weight updates interrupting generation): a request that comes back ``aborted`` is re-issued with
    the tokens produced so far appended to the prompt and the remaining token budget, until it finishes for real."""

    def __init__(self, servers: dict, balancer=None, max_resumes: int = 16, resume_delay_s: float = 0.05):
        super().__init__(servers, balancer)
        self.max_resumes, self.resume_delay_s = max_resumes, resume_delay_s

    async def generate(self, request_id, prompt_ids, sampling_params: Optional[SamplingParams] = None, multi_modal: Optional[dict] = None) -> TokenOutput:
        import dataclasses

        sp = sampling_params or SamplingParams()
        toks: list = []
        lps: list = []
        preempted = 0
        budget = sp.max_tokens
        out = None
        for attempt in range(self.max_resumes + 1):
            cur = dataclasses.replace(sp, max_tokens=budget)
            out = await super().generate(request_id, list(prompt_ids) + toks, cur, multi_modal)
            toks += list(out.token_ids)
            lps += list(out.log_probs or [])
            preempted += out.num_preempted
            budget = sp.max_tokens - len(toks)
            if out.stop_reason != "aborted" or budget <= 0 or self.closed:
                break
            await asyncio.sleep(self.resume_delay_s)
        reason = out.stop_reason if out.stop_reason != "aborted" or budget > 0 else "length"
        return TokenOutput(token_ids=toks, log_probs=lps if sp.logprobs else None, stop_reason=reason, num_preempted=preempted,
                           extra_fields={"resumes": attempt})


class LLMServerManager:
    """The fleet of replicas of one job: ``world_size / (tp·dp·pp)`` of them, a shared load balancer, client factory and
    the Prometheus target list."""

    def __init__(self, replicas: Sequence, fully_async: bool = False):
        self.replicas = list(replicas)
        self.fully_async = fully_async
        self.servers = {f"replica-{r.replica_rank}": (r.server if r.server is not None else r.address) for r in self.replicas}
        self.balancer = GlobalRequestLoadBalancer(list(self.servers))

    @staticmethod
    def num_replicas(world_size: int, tp: int = 1, dp: int = 1, pp: int = 1) -> int:
        per = tp * dp * pp
        assert world_size % per == 0, "world size must be a multiple of tp·dp·pp of one replica"
        return world_size // per

    def client(self) -> LLMServerClient:
        cls = FullyAsyncLLMServerClient if self.fully_async else LLMServerClient
        c = cls(self.servers, self.balancer)
        c.servers = self.servers          # shared, not copied: servers that join or leave later are seen by every client
        return c

    def add_server(self, name: str, target) -> None:
        """Let the balancer route to one more server (an in-process ``AsyncRolloutServer`` or a ``host:port`` address)."""
        self.servers[name] = target
        self.balancer.add_server(name)

    def remove_server(self, name: str) -> None:
        """Stop routing to ``name``. Requests it is still running finish (or are aborted by the caller) under its old entry."""
        self.balancer.remove_server(name)

    def prometheus_targets(self) -> list[str]:
        return [r.address for r in self.replicas if r.address]

    def wake_up(self):
        for r in self.replicas:
            r.wake_up()

    def sleep(self):
        for r in self.replicas:
            r.sleep()

    def abort_all_requests(self):
        for r in self.replicas:
            r.abort_all_requests()

    def shutdown(self):
        for r in self.replicas:
            r.shutdown()
