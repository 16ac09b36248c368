"""The trainer's side of served teachers: score a sequence on the right teacher, cut out and pad the response window.

Reference: ``verl/experimental/teacher_loop/teacher_manager.py:36-144`` (sampling parameters of a scoring request, routing by
``distillation.teacher_key``, padding of the per-sequence outputs to the batch's prompt / response widths).
"""

from __future__ import annotations

import asyncio
import warnings
from typing import Optional, Sequence
from uuid import uuid4

import torch

from verl_b200.workers.rollout.engine import SamplingParams

__all__ = ["teacher_sampling_params", "pad_teacher_outputs", "AsyncTeacherLLMServerManager"]


def teacher_sampling_params(topk: int, use_topk: bool = True, temperature: float = 1.0) -> SamplingParams:
    """A scoring request generates nothing; the temperature has no effect on the log-probs of a forward pass."""
    if temperature != 1.0:
        warnings.warn(f"teacher inference temperature {temperature} has no effect on prompt log-probs; using 1.0", stacklevel=2)
    return SamplingParams(temperature=1.0, max_tokens=1, prompt_logprobs=int(topk) if use_topk else 0)


def pad_teacher_outputs(teacher_ids: torch.Tensor, teacher_logprobs: torch.Tensor, prompt_width: int, response_width: int, prompt_length: int,
                        response_length: int, pad_token_id: int) -> tuple:
    """[L, k] outputs of one unpadded sequence → [1, prompt_width + response_width, k] in the batch layout (prompts left-padded,
    responses right-padded)."""
    if teacher_ids.shape[0] != prompt_length + response_length:
        raise ValueError(f"teacher output has {teacher_ids.shape[0]} rows for a sequence of {prompt_length} + {response_length} tokens")
    pad = (0, 0, prompt_width - prompt_length, response_width - response_length)
    F = torch.nn.functional
    return F.pad(teacher_ids, pad, value=pad_token_id).unsqueeze(0), F.pad(teacher_logprobs, pad, value=0.0).unsqueeze(0)


class AsyncTeacherLLMServerManager:
    """``teacher_client``: ``{routing key: LLMServerClient}``; one key → every sequence goes there, several → the sample's
    ``routing_key`` (the value of ``distillation.teacher_key`` in its non-tensor data) picks the teacher."""

    def __init__(self, distillation_config, teacher_client: dict):
        g = (lambda k, d=None: distillation_config.get(k, d)) if hasattr(distillation_config, "get") else (lambda k, d=None: getattr(distillation_config, k, d))
        self.teacher_key = str(g("teacher_key", "data_source"))
        self.topk = int(g("topk", 32))
        models = g("teacher_models", None) or {}
        expected = set(models) if models else set(teacher_client)
        if set(teacher_client) != expected:
            raise ValueError(f"teacher client keys {sorted(teacher_client)} do not match teacher routing keys {sorted(expected)}.")
        self.teacher_client = dict(teacher_client)
        self.sampling_params = teacher_sampling_params(self.topk, use_topk=self.topk > 0)

    def resolve_teacher_key(self, routing_key: Optional[str]) -> str:
        if len(self.teacher_client) == 1:
            return next(iter(self.teacher_client))
        if routing_key is None:
            raise ValueError(f"Routing key is required for multi-teacher distillation (configured via distillation.teacher_key={self.teacher_key!r}).")
        if routing_key not in self.teacher_client:
            raise ValueError(f"No teacher configured for routing key {routing_key!r}. Configured teachers: {sorted(self.teacher_client)}.")
        return routing_key

    async def compute_teacher_logprobs_single(self, sequence_ids: Sequence[int], routing_key: Optional[str] = None) -> tuple:
        client = self.teacher_client[self.resolve_teacher_key(routing_key)]
        out = await client.generate(uuid4().hex, list(sequence_ids), self.sampling_params)
        ids = torch.tensor(out.extra_fields["prompt_ids"], dtype=torch.int32)
        lps = torch.tensor(out.extra_fields["prompt_logprobs"], dtype=torch.float32)
        if not (ids.shape[0] == lps.shape[0] == len(sequence_ids)):
            raise RuntimeError(f"teacher returned {ids.shape[0]} rows for {len(sequence_ids)} tokens")
        return ids, lps

    async def compute_teacher_topk_async(self, prompts: torch.Tensor, responses: torch.Tensor, attention_mask: torch.Tensor,
                                         routing_keys: Optional[Sequence] = None, pad_token_id: int = 0) -> tuple:
        """Batch front end: ``prompts`` [B, P] (left-padded), ``responses`` [B, R], ``attention_mask`` [B, P + R] →
        ``(teacher_topk_ids [B, R, k], teacher_topk_log_probs [B, R, k])``; rows of padded response positions are zero."""
        B, P = prompts.shape
        R = responses.shape[1]
        seqs, lens = [], []
        for i in range(B):
            pl, rl = int(attention_mask[i, :P].sum()), int(attention_mask[i, P:].sum())
            seqs.append(prompts[i, P - pl:].tolist() + responses[i, :rl].tolist())
            lens.append((pl, rl))
        outs = await asyncio.gather(*[self.compute_teacher_logprobs_single(s, None if routing_keys is None else routing_keys[i]) for i, s in enumerate(seqs)])
        ids_b, lps_b = [], []
        for (ids, lps), (pl, rl) in zip(outs, lens):
            a, b = pad_teacher_outputs(ids, lps, P, R, pl, rl, pad_token_id)
            ids_b.append(a[:, P:])
            lps_b.append(b[:, P:])
        return torch.cat(ids_b).long(), torch.cat(lps_b)

    def compute_teacher_topk(self, *args, **kwargs) -> tuple:
        """Synchronous form for trainers that own no event loop: the HTTP sessions live and die with the loop of this call."""
        async def run():
            try:
                return await self.compute_teacher_topk_async(*args, **kwargs)
            finally:
                for c in self.teacher_client.values():
                    await c.close()

        return asyncio.run(run())
