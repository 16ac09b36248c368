"""DAPO reward: rule score plus a soft penalty for responses that run into the length limit
(reference: ``verl/workers/reward_manager/dapo.py``)."""

from __future__ import annotations

import torch

from verl_b200.protocol import DataProto

from .naive import NaiveRewardManager
from .registry import register


@register("dapo")
class DAPORewardManager(NaiveRewardManager):
    def __init__(self, tokenizer=None, num_examine=0, compute_score=None, reward_fn_key="data_source", max_resp_len=None,
                 overlong_buffer_cfg=None, **kwargs):
        super().__init__(tokenizer, num_examine, compute_score, reward_fn_key)
        self.max_resp_len = max_resp_len
        self.overlong = overlong_buffer_cfg

    def __call__(self, data: DataProto, return_dict: bool = False):
        out = super().__call__(data, return_dict=True)
        reward, extra = out["reward_tensor"], out["reward_extra_info"]
        ob = self.overlong
        if ob is not None and (ob.get("enable", False) if hasattr(ob, "get") else ob.enable):
            assert self.max_resp_len is not None
            buf = ob.get("len") if hasattr(ob, "get") else ob.len
            factor = ob.get("penalty_factor") if hasattr(ob, "get") else ob.penalty_factor
            P = data.batch["prompts"].shape[-1]
            r_lens = data.batch["attention_mask"][:, P:].sum(-1)
            expected = self.max_resp_len - buf
            pen = torch.clamp(-(r_lens - expected).float() / buf * factor, max=0.0)
            idx = (r_lens - 1).clamp(min=0)[:, None]
            reward.scatter_add_(1, idx, pen[:, None] * (r_lens > 0)[:, None].float())
            extra["overlong_reward"] = pen.tolist()
            extra["overlong"] = (pen < 0).tolist()
        return {"reward_tensor": reward, "reward_extra_info": extra} if return_dict else reward
