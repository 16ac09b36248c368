"""One prompt → one completion (reference: ``verl/experimental/agent_loop/single_turn_agent_loop.py:28``)."""

from __future__ import annotations

import time
import uuid

from .agent_loop import AgentLoopBase, AgentLoopMetrics, AgentLoopOutput, register


@register("single_turn_agent")
class SingleTurnAgentLoop(AgentLoopBase):
    async def run(self, sampling_params, **kwargs) -> AgentLoopOutput:
        mm = kwargs.get("multi_modal_inputs") or None      # vision-language prompt: the batch's ids hold the expanded image placeholders
        if kwargs.get("raw_prompt") is not None and self.tokenizer is not None and not (mm and kwargs.get("prompt_ids") is not None):
            prompt_ids = self.chat_ids(list(kwargs["raw_prompt"]))
        else:
            prompt_ids = list(kwargs["prompt_ids"])
        t0 = time.perf_counter()
        out = await (self.client.generate(uuid.uuid4().hex, prompt_ids, sampling_params, mm) if mm
                     else self.client.generate(uuid.uuid4().hex, prompt_ids, sampling_params))
        m = AgentLoopMetrics(generate_sequences=time.perf_counter() - t0, num_preempted=out.num_preempted)
        ids = list(out.token_ids)[: self.response_length]
        return AgentLoopOutput(prompt_ids=prompt_ids, response_ids=ids, response_mask=[1] * len(ids),
                               response_logprobs=list(out.log_probs)[: len(ids)] if out.log_probs is not None else None,
                               num_turns=2, metrics=m)
