"""HTTP router in front of the reward-model (or any generation) servers: one address for the reward-loop workers, requests
spread over the replicas by in-flight count, requests that carry the same ``request_id`` kept on the replica that served
them first (its prefix cache holds their prompt).

Reference: ``verl/experimental/reward_loop/router/naive_router.py:52-205`` (a FastAPI process that forwards every path to
the least-loaded worker). Here the router is an aiohttp application on a background thread of the process that owns the
reward-model manager; the forwarding rule, the endpoints it forwards and the health / worker listing are the same.
"""

from __future__ import annotations

import asyncio
import threading
from collections import OrderedDict
from typing import Optional, Sequence

__all__ = ["NaiveRouter", "RouterClient", "launch_router"]

FORWARDED_POST = ("/generate", "/v1/completions", "/v1/chat/completions", "/score")


class NaiveRouter:
    def __init__(self, worker_urls: Sequence[str], max_sticky: int = 10000, timeout_s: float = 600.0):
        assert worker_urls, "the router needs at least one worker"
        self.worker_urls = [u if u.startswith("http") else f"http://{u}" for u in worker_urls]
        self.inflight = {u: 0 for u in self.worker_urls}
        self.served = {u: 0 for u in self.worker_urls}
        self.sticky: OrderedDict[str, str] = OrderedDict()
        self.max_sticky, self.timeout_s = max_sticky, timeout_s
        self._session = None

    # ------------------------------------------------------------------ worker choice
    def select_worker(self, request_id: Optional[str] = None) -> str:
        if request_id is not None and request_id in self.sticky:
            url = self.sticky[request_id]
            self.sticky.move_to_end(request_id)
        else:
            url = min(self.worker_urls, key=lambda u: (self.inflight[u], self.served[u]))
            if request_id is not None:
                self.sticky[request_id] = url
                while len(self.sticky) > self.max_sticky:
                    self.sticky.popitem(last=False)
        self.inflight[url] += 1
        self.served[url] += 1
        return url

    def release_worker(self, url: str) -> None:
        self.inflight[url] = max(0, self.inflight[url] - 1)

    # ------------------------------------------------------------------ aiohttp application
    def build_app(self):
        import aiohttp
        from aiohttp import web

        async def forward(req: web.Request):
            body = await req.read()
            rid = None
            try:
                import json

                rid = json.loads(body or b"{}").get("request_id")
            except Exception:
                pass
            url = self.select_worker(rid)
            try:
                if self._session is None:
                    self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s))
                async with self._session.post(url + req.path, data=body, headers={"Content-Type": req.headers.get("Content-Type", "application/json")}) as r:
                    payload = await r.read()
                    return web.Response(body=payload, status=r.status, content_type=r.content_type)
            except aiohttp.ClientError as e:
                return web.json_response({"error": f"worker {url} failed: {e}"}, status=502)
            finally:
                self.release_worker(url)

        async def health(_):
            return web.json_response({"status": "ok", "workers": len(self.worker_urls)})

        async def workers(_):
            return web.json_response({"workers": [{"url": u, "inflight": self.inflight[u], "served": self.served[u]} for u in self.worker_urls]})

        async def on_cleanup(_):
            if self._session is not None:
                await self._session.close()

        app = web.Application(client_max_size=256 * 1024 * 1024)
        app.add_routes([web.post(p, forward) for p in FORWARDED_POST] + [web.get("/health", health), web.get("/workers", workers)])
        app.on_cleanup.append(on_cleanup)
        return app


def launch_router(worker_urls: Sequence[str], host: str = "127.0.0.1", port: int = 0):
    """Start a router on a background thread. Returns ``(address, router, stop_fn)``."""
    from aiohttp import web

    router = NaiveRouter(worker_urls)
    loop = asyncio.new_event_loop()
    ready = threading.Event()
    info: dict = {}

    def run():
        asyncio.set_event_loop(loop)
        runner = web.AppRunner(router.build_app())
        loop.run_until_complete(runner.setup())
        site = web.TCPSite(runner, host, port)
        loop.run_until_complete(site.start())
        info["port"] = site._server.sockets[0].getsockname()[1]
        ready.set()
        loop.run_forever()
        loop.run_until_complete(runner.cleanup())

    th = threading.Thread(target=run, name="reward-router", daemon=True)
    th.start()
    if not ready.wait(30):
        raise RuntimeError("the router did not come up within 30 s")

    def stop():
        loop.call_soon_threadsafe(loop.stop)
        th.join(timeout=10)

    return f"{host}:{info['port']}", router, stop


class RouterClient:
    """``generate(request_id, prompt_ids, sampling_params)`` against a router (or a single server) address: the interface the
    reward-loop managers expect from an ``rm_client``."""

    def __init__(self, address: str, timeout_s: float = 600.0):
        self.base = address if address.startswith("http") else f"http://{address}"
        self.timeout_s = timeout_s
        self._sessions: dict = {}

    async def _session(self):
        import aiohttp

        loop = asyncio.get_running_loop()
        s = self._sessions.get(loop)
        if s is None or s.closed:
            s = self._sessions[loop] = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s))
        return s

    async def generate(self, request_id, prompt_ids, sampling_params=None, multi_modal=None):
        from verl_b200.workers.rollout.engine import SamplingParams, TokenOutput

        sp = sampling_params or SamplingParams()
        body = {"prompt_ids": list(prompt_ids), "request_id": request_id,
                "sampling_params": {"temperature": sp.temperature, "top_p": sp.top_p, "top_k": sp.top_k, "max_tokens": sp.max_tokens,
                                    "ignore_eos": sp.ignore_eos, "seed": sp.seed, "stop_token_ids": list(sp.stop_token_ids)}}
        s = await self._session()
        async with s.post(self.base + "/generate", json=body) as r:
            d = await r.json()
            if r.status != 200:
                raise RuntimeError(f"reward-model request failed with {r.status}: {d}")
        out = TokenOutput(token_ids=d["token_ids"], log_probs=d.get("log_probs"), stop_reason=d.get("stop_reason", "length"),
                          num_preempted=d.get("num_preempted", 0))
        if "score" in d:
            out.extra_fields = {"score": d["score"]}
        return out

    async def close(self):
        for s in self._sessions.values():
            if not s.closed:
                await s.close()
        self._sessions.clear()
