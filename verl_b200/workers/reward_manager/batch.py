"""Batched scorer: ``compute_score`` receives lists for the whole batch
(reference: ``verl/workers/reward_manager/batch.py``)."""

from __future__ import annotations

from collections import defaultdict

import torch

from verl_b200.protocol import DataProto

from .naive import NaiveRewardManager
from .registry import register


@register("batch")
class BatchRewardManager(NaiveRewardManager):
    def __call__(self, data: DataProto, return_dict: bool = False):
        if "rm_scores" in data.batch.keys():
            return {"reward_tensor": data.batch["rm_scores"], "reward_extra_info": {}} if return_dict else data.batch["rm_scores"]
        P = data.batch["prompts"].shape[-1]
        att = data.batch["attention_mask"]
        r_lens = att[:, P:].sum(-1)
        texts = [self._decode(data.batch["responses"][i, : int(r_lens[i])]) for i in range(len(data))]
        rm = data.non_tensor_batch.get("reward_model")
        gts = [(x or {}).get("ground_truth") if isinstance(x, dict) else None for x in rm] if rm is not None else [None] * len(data)
        srcs = list(data.non_tensor_batch.get(self.reward_fn_key, ["unknown"] * len(data)))
        extras = list(data.non_tensor_batch.get("extra_info", [None] * len(data)))
        scores = self.compute_score(data_sources=srcs, solution_strs=texts, ground_truths=gts, extra_infos=extras)
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        extra = defaultdict(list)
        for i, s in enumerate(scores):
            if isinstance(s, dict):
                for k, v in s.items():
                    extra[k].append(v)
                s = s["score"]
            if int(r_lens[i]) > 0:
                reward[i, int(r_lens[i]) - 1] = float(s)
        return {"reward_tensor": reward, "reward_extra_info": dict(extra)} if return_dict else reward
