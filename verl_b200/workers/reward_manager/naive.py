"""Per-sample rule reward written at the last valid response token
(reference: ``verl/workers/reward_manager/naive.py``)."""

from __future__ import annotations

from collections import defaultdict

import torch

from verl_b200.protocol import DataProto
from verl_b200.utils.reward_score import default_compute_score

from .registry import register


@register("naive")
class NaiveRewardManager:
    def __init__(self, tokenizer=None, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source", **kwargs):
        self.tokenizer = tokenizer
        self.num_examine = num_examine
        self.compute_score = compute_score or default_compute_score
        self.reward_fn_key = reward_fn_key

    def _decode(self, ids):
        if self.tokenizer is not None:
            return self.tokenizer.decode(ids, skip_special_tokens=True)
        return " ".join(str(int(t)) for t in ids)

    def __call__(self, data: DataProto, return_dict: bool = False):
        if "rm_scores" in data.batch.keys():
            if return_dict:
                return {"reward_tensor": data.batch["rm_scores"], "reward_extra_info": {}}
            return data.batch["rm_scores"]
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        extra = defaultdict(list)
        P = data.batch["prompts"].shape[-1]
        att = data.batch["attention_mask"]
        printed = defaultdict(int)
        for i in range(len(data)):
            p_len = int(att[i, :P].sum())
            r_len = int(att[i, P:].sum())
            prompt_ids = data.batch["prompts"][i, P - p_len:] if p_len else data.batch["prompts"][i, :0]
            resp_ids = data.batch["responses"][i, :r_len]
            nt = {k: v[i] for k, v in data.non_tensor_batch.items()}
            gt = (nt.get("reward_model") or {}).get("ground_truth") if isinstance(nt.get("reward_model"), dict) else nt.get("ground_truth")
            src = nt.get(self.reward_fn_key, "unknown")
            score = self.compute_score(data_source=src, solution_str=self._decode(resp_ids), ground_truth=gt, extra_info=nt.get("extra_info"))
            if isinstance(score, dict):
                for k, v in score.items():
                    extra[k].append(v)
                score = score["score"]
            if r_len > 0:
                reward[i, r_len - 1] = float(score)
            if printed[src] < self.num_examine:
                printed[src] += 1
                print("[prompt]", self._decode(prompt_ids), "\n[response]", self._decode(resp_ids), "\n[ground_truth]", gt, "\n[score]", score)
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": dict(extra)}
        return reward
