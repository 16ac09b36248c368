"""Serving layer, load balancing, agent loops and tools on CPU with the tiny model and a byte-level tokenizer."""

import asyncio
import json
import urllib.request

import numpy as np
import pytest
import torch

from verl_b200.experimental.agent_loop import AgentLoopManager, AgentLoopWorker, get_tool_parser
from verl_b200.models.config import PRESETS
from verl_b200.models.transformer import DecoderLM
from verl_b200.protocol import DataProto
from verl_b200.tools import FunctionTool, initialize_tools_from_config
from verl_b200.utils.config import Config
from verl_b200.utils.tokenizer import ByteChatTokenizer
from verl_b200.workers.rollout.async_server import AsyncRolloutServer, serve_http
from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams, TokenOutput
from verl_b200.workers.rollout.llm_server import FullyAsyncLLMServerClient, GlobalRequestLoadBalancer, LLMServerClient, LLMServerManager
from verl_b200.workers.rollout.replica import RolloutReplica, get_rollout_replica_class


@pytest.fixture(scope="module")
def engine():
    model = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=3)
    return InferenceEngine(model, max_num_seqs=8, max_model_len=256, num_blocks=64)


def _prompts(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(10, 250, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g).tolist() for _ in range(n)]


def test_server_matches_batch_engine_and_serves_http(engine):
    prompts = _prompts(6)
    sp = SamplingParams(temperature=0.0, max_tokens=12)
    want = engine.generate(prompts, sp)
    server = AsyncRolloutServer(engine)
    try:
        futs = [server.submit(p, SamplingParams(temperature=0.0, max_tokens=12 if i % 2 == 0 else 5)) for i, p in enumerate(prompts)]
        outs = [f.result(timeout=120) for f in futs]
        for i, (o, w) in enumerate(zip(outs, want)):
            k = 12 if i % 2 == 0 else 5
            assert o.token_ids == w.token_ids[:k] and o.stop_reason == "length"
            assert np.allclose(o.log_probs, w.log_probs[:k], atol=1e-4)
        addr, stop = serve_http(server)
        try:
            assert json.load(urllib.request.urlopen(f"http://{addr}/health"))["status"] == "ok"
            client = LLMServerClient({"a": addr})

            async def go():
                r = await asyncio.gather(*[client.generate(f"r{i}", p, sp) for i, p in enumerate(prompts[:3])])
                await client.close()
                return r

            for o, w in zip(asyncio.run(go()), want):
                assert o.token_ids == w.token_ids
            text = urllib.request.urlopen(f"http://{addr}/metrics").read().decode()
            assert "verl_b200_rollout_finished" in text
        finally:
            stop()
        assert server.num_inflight == 0
    finally:
        server.shutdown()


def test_abort_returns_partial_output_and_client_resumes(engine):
    server = AsyncRolloutServer(engine)
    try:
        p = _prompts(1)[0]
        sp = SamplingParams(temperature=0.0, max_tokens=150)
        want = engine.generate([p], sp)[0].token_ids
        client = FullyAsyncLLMServerClient({"a": server}, resume_delay_s=0.0)

        async def go():
            task = asyncio.create_task(client.generate("x", p, sp))
            await asyncio.sleep(0.3)
            await asyncio.get_running_loop().run_in_executor(None, server.abort_all_requests)
            return await task

        out = asyncio.run(go())
        assert out.token_ids == want and out.stop_reason == "length"
    finally:
        server.shutdown()


def test_load_balancer_is_sticky_and_prefers_idle_servers():
    lb = GlobalRequestLoadBalancer(["a", "b", "c"], max_cache_size=2)
    first = lb.acquire("req-1")
    others = {lb.acquire(f"req-{i}") for i in (2, 3)}
    assert first not in others and len(others) == 2          # least in-flight spreads the load
    assert lb.acquire("req-3") in others                      # sticky while cached
    for s in ("a", "b", "c"):
        lb.release(s)
    lb.remove_server(first)
    assert lb.acquire("req-9") != first
    assert LLMServerManager.num_replicas(8, tp=2) == 4 and get_rollout_replica_class("vllm") is RolloutReplica


def test_tool_parsers_and_function_tool():
    text = 'I will add.<tool_call>{"name": "add", "arguments": {"a": 2, "b": 3}}</tool_call> ok <tool_call>broken</tool_call>'
    content, calls = get_tool_parser("hermes").extract_tool_calls(text)
    assert [c.name for c in calls] == ["add"] and json.loads(calls[0].arguments) == {"a": 2, "b": 3} and "tool_call" not in content
    _, calls = get_tool_parser("qwen3_xml").extract_tool_calls("<tool_call><function=add><parameter=a>2</parameter><parameter=s>hi</parameter></function></tool_call>")
    assert json.loads(calls[0].arguments) == {"a": 2, "s": "hi"}
    _, calls = get_tool_parser("gpt-oss").extract_tool_calls('<|channel|>commentary to=functions.add <|constrain|>json<|message|>{"a": 1}<|call|>')
    assert calls[0].name == "add"

    def add(a: int, b: int = 1) -> int:
        """Add two integers.

        Args:
            a: first addend
            b: second addend
        """
        return a + b

    tool = FunctionTool(add)
    s = tool.tool_schema.to_dict()["function"]
    assert s["name"] == "add" and s["parameters"]["required"] == ["a"] and s["parameters"]["properties"]["a"] == {"type": "integer", "description": "first addend"}
    resp, _, _ = asyncio.run(tool.execute("i", {"a": 2, "b": 5}))
    assert resp.text == "7"
    resp, _, m = asyncio.run(tool.execute("i", {"zzz": 1}))
    assert "Error" in resp.text and m["tool_error"] == 1
    assert initialize_tools_from_config([{"function": add}])[0].name == "add"


CFG = Config({"rollout": {"prompt_length": 64, "response_length": 48, "temperature": 1.0, "do_sample": False, "free_cache_engine": False,
                          "agent": {"num_workers": 2}, "multi_turn": {"format": "hermes", "max_assistant_turns": 3, "max_tool_response_length": 64}}})


def test_single_turn_agent_loop_equals_plain_generation(engine):
    tok = ByteChatTokenizer()
    prompts = _prompts(5, seed=4)
    want = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=48))
    P = 64
    ids = torch.full((5, P), tok.pad_token_id)
    att = torch.zeros(5, P, dtype=torch.int64)
    for i, p in enumerate(prompts):
        ids[i, P - len(p):] = torch.tensor(p)
        att[i, P - len(p):] = 1
    batch = DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": att}, meta_info={"do_sample": False})
    replica = RolloutReplica(0, CFG).init_hybrid(engine)
    mgr = AgentLoopManager(CFG, LLMServerManager([replica]), tok, reward_fn=lambda **kw: 0.5)
    try:
        out = mgr.generate_sequences(batch)
    finally:
        replica.shutdown()
    for i, w in enumerate(want):
        n = len(w.token_ids)
        assert out.batch["responses"][i, :n].tolist() == w.token_ids and int(out.batch["response_mask"][i].sum()) == n
        assert out.batch["rm_scores"][i, n - 1] == 0.5 and out.batch["rm_scores"][i].sum() == 0.5
        assert torch.equal(out.batch["prompts"][i], ids[i])
    assert out.batch["position_ids"].shape == (5, 112) and "agent_loop/generate_sequences/mean" in out.meta_info["timing"]


class ScriptedClient:
    """Stands in for the servers: first turn asks for a tool, second turn answers."""

    def __init__(self, tok):
        self.tok, self.calls = tok, []

    async def generate(self, request_id, prompt_ids, sp):
        self.calls.append((request_id, list(prompt_ids), sp.max_tokens))
        if len(self.calls) == 1:
            text = 'calling<tool_call>{"name": "add", "arguments": {"a": 20, "b": 22}}</tool_call><|im_end|>'
        else:
            text = "the answer is 42<|im_end|>"
        ids = self.tok.encode(text)
        return TokenOutput(token_ids=ids, log_probs=[-0.5] * len(ids), stop_reason="stop")


def test_tool_agent_loop_masks_tool_tokens():
    tok = ByteChatTokenizer()
    cfg = Config({"rollout": {"prompt_length": 512, "response_length": 400, "agent": {"default_agent_loop": "tool_agent"},
                              "multi_turn": {"format": "hermes", "max_assistant_turns": 4}}})
    client = ScriptedClient(tok)
    worker = AgentLoopWorker(cfg, client, tok, tools=[FunctionTool(lambda a, b: a + b, name="add", description="add")])
    raw = np.empty(1, dtype=object)
    raw[0] = [{"role": "user", "content": "what is 20+22?"}]
    out = worker.generate_sequences(DataProto(batch=None, non_tensor_batch={"raw_prompt": raw}, meta_info={}))
    resp, mask = out.batch["responses"][0], out.batch["response_mask"][0]
    n = int(out.batch["attention_mask"][0, 512:].sum())
    text_model = tok.decode(resp[:n][mask[:n].bool()].tolist())
    text_tool = tok.decode(resp[:n][~mask[:n].bool()].tolist())
    assert "the answer is 42" in text_model and "tool_call" in text_model and "42" in text_tool and "<|im_start|>tool" in text_tool
    assert len(client.calls) == 2 and client.calls[0][0] == client.calls[1][0]            # same sticky request id
    assert client.calls[1][1][: len(client.calls[0][1])] == client.calls[0][1]            # the context only grows
    assert int(out.non_tensor_batch["__num_turns__"][0]) == 4
    assert (out.batch["rollout_log_probs"][0][:n][~mask[:n].bool()] == 0).all()
    assert "Tools" in tok.decode(out.batch["prompts"][0][out.batch["attention_mask"][0, :512].bool()].tolist())


def test_trainer_step_with_server_mode_rollout(tmp_path):
    from tests.test_trainer_e2e_on_cpu import OV, build

    tr = build(tmp_path, ["actor_rollout_ref.rollout.mode=async", "actor_rollout_ref.rollout.prompt_length=32",
                          "actor_rollout_ref.rollout.response_length=16", "actor_rollout_ref.rollout.agent.num_workers=2"])
    m = tr.step(next(iter(tr.train_dataloader)))
    assert m["perf/total_num_tokens"] > 0 and abs(m["actor/ppo_kl"]) < 1e-4 and "timing_s/gen" in m
