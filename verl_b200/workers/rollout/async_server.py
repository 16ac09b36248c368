"""Request-level serving on top of the continuous-batching engine: a server thread that keeps the engine's generation
loop open, futures for callers, and an HTTP front end (token-in/token-out ``/generate``, OpenAI-style
``/v1/completions`` and ``/v1/chat/completions``, ``/health``, ``/metrics``, ``/abort``, ``/sleep``, ``/wake_up``).

Parity target: the reference's per-replica server actors (``verl/workers/rollout/vllm_rollout/vllm_async_server.py:
561-789`` ``generate`` → ``TokenOutput``; ``wake_up/sleep/abort_all_requests/resume``), with the in-house engine in place
of vLLM's ``AsyncLLM``.
"""

from __future__ import annotations

import asyncio
import concurrent.futures
import dataclasses
import json
import queue
import threading
import time
from typing import Optional

from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams, TokenOutput

__all__ = ["AsyncRolloutServer", "build_http_app", "serve_http"]


def _sp_key(sp: SamplingParams):
    d = dataclasses.asdict(sp)
    d.pop("max_tokens", None)
    d["stop_token_ids"] = tuple(d.get("stop_token_ids") or ())
    return tuple(sorted(d.items()))


class AsyncRolloutServer:
    """Owns one ``InferenceEngine``; ``submit`` may be called from any thread (or ``await generate`` from asyncio).

    Requests whose sampling parameters (apart from ``max_tokens``) equal those of the running batch join it at the
    engine's next synchronisation point; others wait until the batch has drained.
    """

    def __init__(self, engine: InferenceEngine, eos_token_id=None, tokenizer=None, name: str = "replica-0"):
        self.engine, self.eos_token_id, self.tokenizer, self.name = engine, eos_token_id, tokenizer, name
        self._q: "queue.Queue[tuple]" = queue.Queue()
        self._held: list[tuple] = []
        self._stop = threading.Event()
        self._abort = threading.Event()
        self._paused = threading.Event()
        self._idle = threading.Event()
        self._idle.set()
        self.stats = {"requests": 0, "finished": 0, "aborted": 0, "generated_tokens": 0, "prompt_tokens": 0, "busy_s": 0.0}
        self._thread = threading.Thread(target=self._loop, name=f"rollout-{name}", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ client side
    def submit(self, prompt_ids, sampling_params: Optional[SamplingParams] = None, request_id: Optional[str] = None,
               multi_modal: Optional[dict] = None) -> concurrent.futures.Future:
        """``multi_modal``: ``{"pixel_values", "image_grid_thw"}`` of a vision-language prompt (its placeholders already expanded)."""
        fut: concurrent.futures.Future = concurrent.futures.Future()
        sp = sampling_params or SamplingParams()
        self.stats["requests"] += 1
        self.stats["prompt_tokens"] += len(prompt_ids)
        self._q.put((list(prompt_ids), sp, fut, request_id, multi_modal))
        return fut

    async def generate(self, prompt_ids, sampling_params: Optional[SamplingParams] = None, request_id: Optional[str] = None,
                       multi_modal: Optional[dict] = None) -> TokenOutput:
        return await asyncio.wrap_future(self.submit(prompt_ids, sampling_params, request_id, multi_modal))

    @property
    def num_inflight(self) -> int:
        return self.stats["requests"] - self.stats["finished"] - self.stats["aborted"]

    def abort_all_requests(self) -> None:
        """Finish every running request now with its partial output (``stop_reason="aborted"``); queued ones too."""
        self._abort.set()
        self._idle.wait(timeout=60)
        self._abort.clear()

    def pause(self):
        """Stop admitting queued requests (weight update in progress); running ones finish or are aborted separately."""
        self._paused.set()

    def resume(self):
        self._paused.clear()

    def wait_idle(self, timeout: float = 600.0) -> bool:
        return self._idle.wait(timeout)

    def sleep(self):
        self.wait_idle()
        self.engine.sleep()

    def wake_up(self):
        self.engine.wake_up()

    def shutdown(self):
        self._stop.set()
        self._thread.join(timeout=30)

    # ------------------------------------------------------------------ weight hand-off (replicas on their own GPUs)
    def update_weights(self, source: dict) -> int:
        """Replace the model weights of this replica from ``source`` and return the new weights version.

        The running batch is interrupted (its requests come back ``aborted`` with their partial output, resumable clients
        continue them under the new weights), admission is paused while the copy runs. ``source`` describes a flat parameter
        buffer and its layout (``names / shapes / offsets``):

        * ``{"kind": "cuda_ipc", "handle": <base64 CUDA IPC handle>, "nbytes": n, "dtype": "bfloat16", ...}`` — the trainer's
          export buffer on another GPU of this machine; it is mapped here and copied device-to-device over NVLink;
        * ``{"kind": "file", "path": p, ...}`` — a ``torch.save``d dict holding ``flat`` (CPU path, also the fallback).
        """
        import base64

        import torch

        self.pause()
        try:
            self.abort_all_requests()
            self.wait_idle()
            params = dict(self.engine.model.named_parameters())
            opened = None
            if source["kind"] == "cuda_ipc":
                from verl_b200.ops import _ext

                ops_ = _ext.ops()
                hb = torch.frombuffer(bytearray(base64.b64decode(source["handle"])), dtype=torch.uint8)
                opened = int(ops_.ipc_open_handle(hb))
                dt = getattr(torch, source.get("dtype", "bfloat16"))
                dev = next(iter(params.values())).device
                # one DMA transfer into local memory; the per-tensor copies below then read this GPU's own memory
                flat = torch.empty(int(source["nbytes"]) // torch.empty(0, dtype=dt).element_size(), dtype=dt, device=dev)
                ops_.peer_memcpy(flat, opened, int(source["nbytes"]))
                torch.cuda.synchronize()
                ops_.ipc_close(opened)
                opened = None
                layout = source
            elif source["kind"] == "file":
                layout = torch.load(source["path"], map_location="cpu", weights_only=False)
                flat = layout["flat"]
            else:
                raise ValueError(f"unknown weight source kind {source['kind']!r}")
            with torch.no_grad():
                for name, shape, off in zip(layout["names"], layout["shapes"], layout["offsets"]):
                    n = 1
                    for d in shape:
                        n *= int(d)
                    params[name].copy_(flat[int(off): int(off) + n].view(*[int(d) for d in shape]))
            if opened is not None:
                ops_.ipc_close(opened)
            self.weights_version = getattr(self, "weights_version", 0) + 1
        finally:
            self.resume()
        return self.weights_version

    def weights_checksum(self) -> float:
        import torch

        with torch.no_grad():
            return float(sum(p.double().sum() for p in self.engine.model.parameters()))

    # ------------------------------------------------------------------ server thread
    def _take(self, key) -> list[tuple]:
        """Queued requests compatible with ``key`` (everything else is held back for the next batch)."""
        out, keep = [], []
        while True:
            try:
                self._held.append(self._q.get_nowait())
            except queue.Empty:
                break
        for item in self._held:
            (out if _sp_key(item[1]) == key else keep).append(item)
        self._held = keep
        return out

    def _loop(self):
        while not self._stop.is_set():
            if self._paused.is_set() or (not self._held and self._q.empty()):
                if self._abort.is_set() and (self._held or not self._q.empty()):
                    self._fail_queued()
                time.sleep(0.001)
                continue
            if not self._held:
                try:
                    self._held.append(self._q.get(timeout=0.05))
                except queue.Empty:
                    continue
            sp = self._held[0][1]
            key = _sp_key(sp)
            futs: list[concurrent.futures.Future] = []
            if getattr(sp, "prompt_logprobs", -1) >= 0:
                self._score(self._take(key), int(sp.prompt_logprobs))
                continue

            def admit():
                if self._paused.is_set():
                    return []
                items = self._take(key)
                futs.extend(it[2] for it in items)
                return [(it[0], it[1].max_tokens, it[4] if len(it) > 4 else None) for it in items]

            def on_done(i, out: TokenOutput):
                self.stats["aborted" if out.stop_reason == "aborted" else "finished"] += 1
                self.stats["generated_tokens"] += len(out.token_ids)
                if not futs[i].done():
                    futs[i].set_result(out)

            self._idle.clear()
            t0 = time.perf_counter()
            try:
                self.engine.generate([], sp, eos_token_id=self.eos_token_id, admit=admit, on_done=on_done,
                                     keep_alive=lambda: False, should_abort=self._abort.is_set)
            except Exception as e:  # noqa: BLE001 - hand the failure to every waiting caller
                for f in futs:
                    if not f.done():
                        f.set_exception(e)
            self.stats["busy_s"] += time.perf_counter() - t0
            if self._abort.is_set():
                self._fail_queued()
            self._idle.set()

    def _score(self, items: list, k: int) -> None:
        """Teacher-style requests: no generation, the per-position (top-k) log-probs of the sequences themselves."""
        self._idle.clear()
        t0 = time.perf_counter()
        try:
            res = self.engine.score_prompts([it[0] for it in items], k)
            for it, (ids, lps) in zip(items, res):
                self.stats["finished"] += 1
                it[2].set_result(TokenOutput(token_ids=[], log_probs=[], stop_reason="scored",
                                             extra_fields={"prompt_ids": ids.tolist(), "prompt_logprobs": lps.tolist()}))
        except Exception as e:  # noqa: BLE001
            for it in items:
                if not it[2].done():
                    it[2].set_exception(e)
        self.stats["busy_s"] += time.perf_counter() - t0
        self._idle.set()

    def _fail_queued(self):
        for item in self._take(None) + self._held:
            self.stats["aborted"] += 1
            item[2].set_result(TokenOutput(token_ids=[], log_probs=[], stop_reason="aborted"))
        self._held = []


# ---------------------------------------------------------------------------------------------------- HTTP front end
def build_http_app(server: AsyncRolloutServer):
    from aiohttp import web

    def _sp(body: dict) -> SamplingParams:
        p = body.get("sampling_params", body)
        return SamplingParams(temperature=float(p.get("temperature", 1.0)), top_p=float(p.get("top_p", 1.0)), top_k=int(p.get("top_k", -1)),
                              max_tokens=int(p.get("max_tokens", p.get("max_new_tokens", 256))), ignore_eos=bool(p.get("ignore_eos", False)),
                              seed=int(p.get("seed", 0) or 0), stop_token_ids=tuple(p.get("stop_token_ids", ()) or ()),
                              prompt_logprobs=int(-1 if p.get("prompt_logprobs") is None else p.get("prompt_logprobs")))

    async def generate(req):
        body = await req.json()
        out = await server.generate(body["prompt_ids"], _sp(body), body.get("request_id"))
        return web.json_response({"token_ids": out.token_ids, "log_probs": out.log_probs, "stop_reason": out.stop_reason,
                                  "num_preempted": out.num_preempted, "extra_fields": out.extra_fields or {}})

    def _need_tok():
        if server.tokenizer is None:
            raise web.HTTPBadRequest(text="this server was started without a tokenizer; use /generate with token ids")

    async def completions(req):
        _need_tok()
        body = await req.json()
        ids = server.tokenizer(body["prompt"], add_special_tokens=False)["input_ids"]
        out = await server.generate(ids, _sp(body))
        text = server.tokenizer.decode(out.token_ids, skip_special_tokens=True)
        return web.json_response({"object": "text_completion", "model": body.get("model", server.name),
                                  "choices": [{"index": 0, "text": text, "finish_reason": out.stop_reason}],
                                  "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out.token_ids)}})

    async def chat(req):
        _need_tok()
        body = await req.json()
        ids = server.tokenizer.apply_chat_template(body["messages"], add_generation_prompt=True, tokenize=True)
        ids = ids["input_ids"] if isinstance(ids, dict) else list(ids)
        n = int(body.get("n", 1))
        outs = await asyncio.gather(*[server.generate(ids, _sp(body)) for _ in range(n)])
        choices = [{"index": i, "message": {"role": "assistant", "content": server.tokenizer.decode(o.token_ids, skip_special_tokens=True)},
                    "finish_reason": o.stop_reason} for i, o in enumerate(outs)]
        return web.json_response({"object": "chat.completion", "model": body.get("model", server.name), "choices": choices,
                                  "usage": {"prompt_tokens": len(ids), "completion_tokens": sum(len(o.token_ids) for o in outs)}})

    async def health(_):
        return web.json_response({"status": "ok", "name": server.name, "inflight": server.num_inflight})

    async def metrics(_):
        st = server.stats
        lines = [f'verl_b200_rollout_{k}{{replica="{server.name}"}} {v}' for k, v in st.items()]
        lines.append(f'verl_b200_rollout_inflight{{replica="{server.name}"}} {server.num_inflight}')
        return web.Response(text="\n".join(lines) + "\n", content_type="text/plain")

    async def abort(_):
        await asyncio.get_running_loop().run_in_executor(None, server.abort_all_requests)
        return web.json_response({"status": "aborted"})

    async def update_weights(req):
        body = await req.json()
        v = await asyncio.get_running_loop().run_in_executor(None, server.update_weights, body)
        return web.json_response({"status": "ok", "weights_version": v})

    async def weights_version(req):
        d = {"weights_version": getattr(server, "weights_version", 0)}
        if req.query.get("checksum"):
            d["checksum"] = await asyncio.get_running_loop().run_in_executor(None, server.weights_checksum)
        return web.json_response(d)

    async def sleep(_):
        await asyncio.get_running_loop().run_in_executor(None, server.sleep)
        return web.json_response({"status": "sleeping"})

    async def wake(_):
        await asyncio.get_running_loop().run_in_executor(None, server.wake_up)
        return web.json_response({"status": "awake"})

    app = web.Application(client_max_size=256 * 1024 * 1024)
    app.add_routes([web.post("/generate", generate), web.post("/v1/completions", completions), web.post("/v1/chat/completions", chat),
                    web.get("/health", health), web.get("/metrics", metrics), web.post("/abort", abort), web.post("/sleep", sleep),
                    web.post("/wake_up", wake), web.post("/update_weights", update_weights), web.get("/weights_version", weights_version)])
    return app


def serve_http(server: AsyncRolloutServer, host: str = "127.0.0.1", port: int = 0):
    """Start the HTTP front end on a background thread; returns ``(address, stop_fn)``."""
    from aiohttp import web

    loop = asyncio.new_event_loop()
    ready = threading.Event()
    info: dict = {}

    def run():
        asyncio.set_event_loop(loop)
        runner = web.AppRunner(build_http_app(server))
        loop.run_until_complete(runner.setup())
        site = web.TCPSite(runner, host, port)
        loop.run_until_complete(site.start())
        info["port"] = site._server.sockets[0].getsockname()[1]
        info["runner"] = runner
        ready.set()
        loop.run_forever()
        loop.run_until_complete(runner.cleanup())

    th = threading.Thread(target=run, name=f"http-{server.name}", daemon=True)
    th.start()
    ready.wait(30)

    def stop():
        loop.call_soon_threadsafe(loop.stop)
        th.join(timeout=10)

    return f"{host}:{info['port']}", stop
