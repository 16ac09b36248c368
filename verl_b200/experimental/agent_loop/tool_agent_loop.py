"""Multi-turn tool-calling loop as a small state machine (reference: ``verl/experimental/agent_loop/tool_agent_loop.py:102``).

PENDING → GENERATING → (tool calls found) PROCESSING_TOOLS → GENERATING → … → TERMINATED. Model tokens carry
``response_mask`` 1, tool-response tokens 0 (and log-prob 0). Limits: assistant turns, user/tool turns, parallel calls per
turn, tool response length, total response length.
"""

from __future__ import annotations

import asyncio
import enum
import json
import time
import uuid

from verl_b200.tools.schemas import OpenAIFunctionCallSchema

from .agent_loop import AgentLoopBase, AgentLoopMetrics, AgentLoopOutput, cfg_get, register
from .tool_parser import get_tool_parser


class AgentState(enum.Enum):
    PENDING = "pending"
    GENERATING = "generating"
    PROCESSING_TOOLS = "processing_tools"
    TERMINATED = "terminated"


@register("tool_agent")
class ToolAgentLoop(AgentLoopBase):
    def __init__(self, config, client, tokenizer, tools=None, **kwargs):
        super().__init__(config, client, tokenizer, tools, **kwargs)
        mt = cfg_get(config, "rollout.multi_turn", {}) or {}
        self.max_assistant_turns = int(cfg_get(mt, "max_assistant_turns", None) or 8)
        self.max_user_turns = int(cfg_get(mt, "max_user_turns", None) or 8)
        self.max_parallel_calls = int(cfg_get(mt, "max_parallel_calls", 1) or 1)
        self.max_tool_response_length = int(cfg_get(mt, "max_tool_response_length", 256) or 256)
        self.truncate_side = cfg_get(mt, "tool_response_truncate_side", "middle")
        self.parser = get_tool_parser(cfg_get(mt, "format", "hermes"), tokenizer)
        self.tool_schemas = [t.tool_schema.to_dict() for t in self.tools.values()]
        from verl_b200.utils.continuous_token import ContinuousTokenBuilder

        self._builder = ContinuousTokenBuilder(self.tokenizer)

    def _truncate(self, text: str) -> str:
        L = self.max_tool_response_length
        if len(text) <= L:
            return text
        if self.truncate_side == "left":
            return text[:L] + "...(truncated)"
        if self.truncate_side == "right":
            return "(truncated)..." + text[-L:]
        return text[: L // 2] + "...(truncated)..." + text[-L // 2:]

    def _tool_turn_ids(self, tool_messages: list) -> list:
        """Tokens that the chat template adds for the tool messages plus the next assistant header."""
        return self._builder.merge_context_tokens([], tool_messages)

    async def _call_tool(self, call, tool_kwargs: dict):
        tool = self.tools.get(call.name)
        if tool is None:
            return f"Error: unknown tool {call.name!r}", 0.0
        parsed, bad = OpenAIFunctionCallSchema.from_openai_function_parsed_schema(call.name, call.arguments)
        if bad:
            return "Error: tool arguments are not valid JSON", 0.0
        kw = (tool_kwargs or {}).get(call.name, {})
        iid, _ = await tool.create(**kw.get("create_kwargs", {}))
        try:
            resp, reward, _ = await tool.execute(iid, parsed.arguments, **kw.get("execute_kwargs", {}))
        finally:
            await tool.release(iid)
        return self._truncate(resp.text or ""), float(reward or 0.0)

    async def run(self, sampling_params, **kwargs) -> AgentLoopOutput:
        # template families whose tool turn does not end with EOS add their own stop token (e.g. <|observation|>, <tool_call|>)
        stop_ids = tuple(sampling_params.stop_token_ids) + tuple(self.parser.stop_token_ids)
        import dataclasses

        messages = list(kwargs["raw_prompt"])
        prompt_ids = self.chat_ids(messages, tools=self.tool_schemas or None)
        request_id = uuid.uuid4().hex
        m = AgentLoopMetrics()
        resp_ids, mask, lps = [], [], []
        state, a_turns, u_turns, tool_reward = AgentState.GENERATING, 0, 0, 0.0
        calls = []
        while state != AgentState.TERMINATED:
            if state == AgentState.GENERATING:
                budget = self.response_length - len(resp_ids)
                if budget <= 0 or a_turns >= self.max_assistant_turns:
                    break
                t0 = time.perf_counter()
                out = await self.client.generate(request_id, prompt_ids + resp_ids, dataclasses.replace(sampling_params, max_tokens=budget, stop_token_ids=stop_ids))
                m.generate_sequences += time.perf_counter() - t0
                m.num_preempted += out.num_preempted
                a_turns += 1
                ids = list(out.token_ids)
                resp_ids += ids
                mask += [1] * len(ids)
                lps += list(out.log_probs) if out.log_probs is not None else [0.0] * len(ids)
                _, calls = self.parser.extract_tool_calls(self.tokenizer.decode(ids))
                if calls and self.tools and u_turns < self.max_user_turns and len(resp_ids) < self.response_length:
                    state = AgentState.PROCESSING_TOOLS
                else:
                    state = AgentState.TERMINATED
            elif state == AgentState.PROCESSING_TOOLS:
                t0 = time.perf_counter()
                results = await asyncio.gather(*[self._call_tool(c, kwargs.get("tools_kwargs") or {}) for c in calls[: self.max_parallel_calls]])
                m.tool_calls += time.perf_counter() - t0
                tool_reward += sum(r for _, r in results)
                tool_ids = self._tool_turn_ids([{"role": "tool", "content": text} for text, _ in results])
                if len(resp_ids) + len(tool_ids) >= self.response_length:
                    state = AgentState.TERMINATED
                    continue
                resp_ids += tool_ids
                mask += [0] * len(tool_ids)
                lps += [0.0] * len(tool_ids)
                u_turns += 1
                state = AgentState.GENERATING
        resp_ids, mask, lps = resp_ids[: self.response_length], mask[: self.response_length], lps[: self.response_length]
        return AgentLoopOutput(prompt_ids=prompt_ids, response_ids=resp_ids, response_mask=mask, response_logprobs=lps,
                               num_turns=1 + a_turns + u_turns, metrics=m, extra_fields={"tool_rewards": tool_reward})
