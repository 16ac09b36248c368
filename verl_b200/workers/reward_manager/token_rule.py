"""Reward computed directly from token ids (no detokenisation): the synthetic mod-7 rule of the benchmark configs,
vectorised over the batch."""

from __future__ import annotations

import torch

from verl_b200.protocol import DataProto

from .registry import register


@register("token_rule")
class TokenRuleRewardManager:
    def __init__(self, tokenizer=None, num_examine: int = 0, compute_score=None, **kwargs):
        self.modulus = int(kwargs.get("modulus", 7))

    def __call__(self, data: DataProto, return_dict: bool = False):
        prompts, resp, att = data.batch["prompts"], data.batch["responses"], data.batch["attention_mask"]
        P = prompts.shape[-1]
        pmask, rmask = att[:, :P], att[:, P:]
        target = (prompts * pmask).sum(-1) % self.modulus
        r_len = rmask.sum(-1)
        last = resp.gather(1, (r_len - 1).clamp(min=0)[:, None]).squeeze(1)
        score = ((last % self.modulus) == target).float() * (r_len > 0).float()
        reward = torch.zeros_like(resp, dtype=torch.float32)
        reward.scatter_(1, (r_len - 1).clamp(min=0)[:, None], score[:, None])
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": {"acc": score.tolist()}}
        return reward
