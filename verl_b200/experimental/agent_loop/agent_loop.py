"""Agent loops: per-sample asyncio tasks that talk to the rollout servers, possibly over several turns with tools, and
are packed back into the trainer's batch layout.

Reference: ``verl/experimental/agent_loop/agent_loop.py`` — ``AgentLoopOutput`` (:88-227), ``AgentLoopBase`` (:227),
``AgentLoopWorker`` (:584-1165: per-sample tasks, left-pad prompt / right-pad response, ``response_mask`` 1 = model token
0 = tool/pad, ``rm_scores`` at the last valid token) and ``AgentLoopManager`` (:1190-1312: chunk over workers, wake/sleep
replicas, timing metrics).
"""

from __future__ import annotations

import asyncio
import time
import uuid
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import numpy as np
import torch

from verl_b200.protocol import DataProto, TensorBatch
from verl_b200.utils.torch_functional import compute_position_id_with_mask
from verl_b200.workers.rollout.engine import SamplingParams

__all__ = ["AgentLoopMetrics", "AgentLoopOutput", "AgentLoopBase", "AgentLoopWorker", "AgentLoopManager", "register", "get_agent_loop_class"]

_AGENT_LOOPS: dict[str, type] = {}


def register(name: str):
    def deco(cls):
        _AGENT_LOOPS[name] = cls
        return cls

    return deco


def get_agent_loop_class(name: str):
    if name not in _AGENT_LOOPS:
        from . import single_turn_agent_loop, tool_agent_loop  # noqa: F401 - populate the registry

    if name not in _AGENT_LOOPS:
        raise ValueError(f"unknown agent loop {name!r}; known: {sorted(_AGENT_LOOPS)}")
    return _AGENT_LOOPS[name]


@dataclass
class AgentLoopMetrics:
    generate_sequences: float = 0.0
    tool_calls: float = 0.0
    num_preempted: int = 0


@dataclass
class AgentLoopOutput:
    prompt_ids: list
    response_ids: list
    response_mask: list                       # 1 = sampled by the model, 0 = injected (tool / user turn)
    response_logprobs: Optional[list] = None
    reward_score: Optional[float] = None
    num_turns: int = 0
    metrics: AgentLoopMetrics = field(default_factory=AgentLoopMetrics)
    extra_fields: dict = field(default_factory=dict)


def cfg_get(cfg, key, default=None):
    cur = cfg
    for part in key.split("."):
        if cur is None:
            return default
        cur = cur.get(part, None) if hasattr(cur, "get") else getattr(cur, part, None)
    return default if cur is None else cur


class AgentLoopBase(ABC):
    """One instance per trajectory. ``client.generate(request_id, prompt_ids, SamplingParams)`` reaches the servers."""

    def __init__(self, config, client, tokenizer, tools: Optional[list] = None, **kwargs):
        self.config, self.client, self.tokenizer = config, client, tokenizer
        self.tools = {t.name: t for t in (tools or [])}
        self.prompt_length = int(cfg_get(config, "rollout.prompt_length", 512))
        self.response_length = int(cfg_get(config, "rollout.response_length", 512))

    def chat_ids(self, messages, tools=None) -> list:
        ids = self.tokenizer.apply_chat_template(messages, tools=tools, add_generation_prompt=True, tokenize=True)
        return list(ids["input_ids"] if isinstance(ids, dict) else ids)

    @abstractmethod
    async def run(self, sampling_params: SamplingParams, **kwargs) -> AgentLoopOutput:
        ...


class AgentLoopWorker:
    """Runs the agent loops of one chunk of the batch concurrently and packs them into tensors."""

    def __init__(self, config, client, tokenizer, tools: Optional[list] = None, reward_fn: Optional[Callable] = None):
        self.config, self.client, self.tokenizer, self.tools, self.reward_fn = config, client, tokenizer, tools or [], reward_fn
        self.prompt_length = int(cfg_get(config, "rollout.prompt_length", 512))
        self.response_length = int(cfg_get(config, "rollout.response_length", 512))
        self.default_agent = cfg_get(config, "rollout.agent.default_agent_loop", "single_turn_agent")

    def _sampling_params(self, meta: dict) -> SamplingParams:
        ro = cfg_get(self.config, "rollout", {})
        validate = bool(meta.get("validate", False))
        vk = cfg_get(ro, "val_kwargs", {}) or {}
        src = vk if validate else ro
        do_sample = bool(cfg_get(src, "do_sample", True)) if validate else bool(meta.get("do_sample", cfg_get(ro, "do_sample", True)))
        temperature = float(meta.get("temperature", cfg_get(src, "temperature", 1.0)))
        return SamplingParams(temperature=temperature if do_sample else 0.0, top_p=float(cfg_get(src, "top_p", 1.0)),
                              top_k=int(cfg_get(src, "top_k", -1)), max_tokens=self.response_length,
                              seed=int(meta.get("seed", 0)) + int(meta.get("global_steps", 0)))

    async def _run_one(self, sp: SamplingParams, sample: dict) -> AgentLoopOutput:
        name = sample.get("agent_name") or self.default_agent
        loop = get_agent_loop_class(str(name))(self.config, self.client, self.tokenizer, tools=self.tools)
        out = await loop.run(sp, **sample)
        if out.reward_score is None and self.reward_fn is not None:
            text = self.tokenizer.decode(out.response_ids, skip_special_tokens=True) if self.tokenizer is not None else ""
            rm = sample.get("reward_model") or {}
            res = self.reward_fn(data_source=sample.get("data_source"), solution_str=text, ground_truth=rm.get("ground_truth") if isinstance(rm, dict) else None,
                                 extra_info=sample.get("extra_info"))
            if asyncio.iscoroutine(res):
                res = await res
            out.reward_score = float(res["score"] if isinstance(res, dict) else res)
        return out

    async def generate_sequences_async(self, batch: DataProto) -> DataProto:
        sp = self._sampling_params(batch.meta_info)
        n = len(batch)
        ntb = batch.non_tensor_batch
        samples = []
        for i in range(n):
            s = {k: v[i] for k, v in ntb.items()}
            if ("raw_prompt" not in s or s.get("multi_modal_inputs")) and batch.batch is not None and "input_ids" in batch.batch:
                att = batch.batch["attention_mask"][i].bool()
                s["prompt_ids"] = batch.batch["input_ids"][i][att].tolist()
            samples.append(s)
        outs = await asyncio.gather(*[self._run_one(sp, s) for s in samples])
        return self._postprocess(outs, batch)

    def generate_sequences(self, batch: DataProto) -> DataProto:
        return asyncio.run(self.generate_sequences_async(batch))

    # ------------------------------------------------------------------ packing
    def _postprocess(self, outs: list[AgentLoopOutput], batch: DataProto) -> DataProto:
        P, R, n = self.prompt_length, self.response_length, len(outs)
        pad = int(getattr(self.tokenizer, "pad_token_id", 0) or 0) if self.tokenizer is not None else int(batch.meta_info.get("pad_token_id", 0) or 0)
        prompts = torch.full((n, P), pad, dtype=torch.int64)
        p_att = torch.zeros(n, P, dtype=torch.int64)
        resp = torch.full((n, R), pad, dtype=torch.int64)
        r_att = torch.zeros(n, R, dtype=torch.int64)
        r_mask = torch.zeros(n, R, dtype=torch.int64)
        lps = torch.zeros(n, R, dtype=torch.float32)
        scores = torch.zeros(n, R, dtype=torch.float32)
        have_score = any(o.reward_score is not None for o in outs)
        for i, o in enumerate(outs):
            p = list(o.prompt_ids)[-P:]
            prompts[i, P - len(p):] = torch.tensor(p, dtype=torch.int64)
            p_att[i, P - len(p):] = 1
            r = list(o.response_ids)[:R]
            k = len(r)
            resp[i, :k] = torch.tensor(r, dtype=torch.int64)
            r_att[i, :k] = 1
            r_mask[i, :k] = torch.tensor(list(o.response_mask)[:k], dtype=torch.int64)
            if o.response_logprobs is not None:
                lps[i, :k] = torch.tensor(list(o.response_logprobs)[:k], dtype=torch.float32)
            if o.reward_score is not None and k > 0:
                scores[i, k - 1] = float(o.reward_score)
        att = torch.cat([p_att, r_att], 1)
        tensors = {"prompts": prompts, "responses": resp, "input_ids": torch.cat([prompts, resp], 1), "attention_mask": att,
                   "position_ids": compute_position_id_with_mask(att), "response_mask": r_mask, "rollout_log_probs": lps}
        if have_score:
            tensors["rm_scores"] = scores
        non_tensor = dict(batch.non_tensor_batch)
        non_tensor["__num_turns__"] = np.array([o.num_turns for o in outs], dtype=np.int32)
        extra_keys = set().union(*[o.extra_fields.keys() for o in outs]) if outs else set()
        for k in extra_keys:
            arr = np.empty(n, dtype=object)
            for i, o in enumerate(outs):
                arr[i] = o.extra_fields.get(k)
            non_tensor[k] = arr
        metrics = [{"generate_sequences": o.metrics.generate_sequences, "tool_calls": o.metrics.tool_calls, "num_preempted": o.metrics.num_preempted}
                   for o in outs]
        return DataProto(batch=TensorBatch(tensors, batch_size=(n,)), non_tensor_batch=non_tensor, meta_info={"agent_metrics": metrics})


class AgentLoopManager:
    """Entry point used by the trainer in place of the plain ``generate_sequences`` RPC when rollouts are agentic.

    ``server_manager`` is an ``LLMServerManager`` (fleet of replicas); the batch is split into ``num_workers`` chunks
    that run concurrently on one event loop (the work is awaiting servers, not computing)."""

    def __init__(self, config, server_manager, tokenizer, tools: Optional[list] = None, reward_fn: Optional[Callable] = None):
        self.config, self.server_manager, self.tokenizer = config, server_manager, tokenizer
        self.num_workers = max(1, int(cfg_get(config, "rollout.agent.num_workers", 8)))
        tool_cfg = cfg_get(config, "rollout.multi_turn.tool_config_path", None)
        if tools is None and tool_cfg:
            from verl_b200.tools import initialize_tools_from_config

            tools = initialize_tools_from_config(tool_cfg)
        self.workers = [AgentLoopWorker(config, server_manager.client(), tokenizer, tools, reward_fn) for _ in range(self.num_workers)]
        self.free_cache = bool(cfg_get(config, "rollout.free_cache_engine", True))

    async def _run(self, chunks):
        return await asyncio.gather(*[w.generate_sequences_async(c) for w, c in zip(self.workers, chunks)])

    def generate_sequences(self, prompts: DataProto) -> DataProto:
        t0 = time.perf_counter()
        self.server_manager.wake_up()
        n = len(prompts)
        k = min(self.num_workers, n)
        bounds = [round(i * n / k) for i in range(k + 1)]
        chunks = [prompts[bounds[i]: bounds[i + 1]] for i in range(k)]
        for c in chunks:
            c.meta_info = dict(prompts.meta_info)
        outs = asyncio.run(self._run(chunks))
        if self.free_cache:
            self.server_manager.sleep()
        ms = [m for o in outs for m in o.meta_info.pop("agent_metrics", [])]
        out = DataProto.concat(outs)
        g = np.array([m["generate_sequences"] for m in ms]) if ms else np.zeros(1)
        t = np.array([m["tool_calls"] for m in ms]) if ms else np.zeros(1)
        timing = {"agent_loop/generate_sequences/min": float(g.min()), "agent_loop/generate_sequences/max": float(g.max()),
                  "agent_loop/generate_sequences/mean": float(g.mean()), "agent_loop/tool_calls/min": float(t.min()),
                  "agent_loop/tool_calls/max": float(t.max()), "agent_loop/tool_calls/mean": float(t.mean()),
                  "generate_sequences": time.perf_counter() - t0}
        n_tok = int(out.batch["response_mask"].sum())
        out.meta_info = {"timing": timing, "metrics": [{"rollout/tokens_per_s": n_tok / max(timing["generate_sequences"], 1e-9)}]}
        return out
