"""Tool-use reward of the ToolRL / GDPO recipes: a format term (does the reply have exactly the blocks the reference answer
has — ``<think>`` then ``<tool_call>`` and / or ``<response>``) plus a tool-call correctness term in ``[-3, 3]`` (tool names,
parameter names and parameter values matched against the reference calls, each reference call paired with its best unused
predicted call). Returns ``{"score", "format_reward", "accuracy_reward"}``, which the GDPO advantage estimator normalises
per reward component.

Behaviour matches ``verl/utils/reward_score/rlla.py`` (format rules :46-100, matching :103-152, score :203-248).
"""

from __future__ import annotations

import json
import re
from collections import Counter

__all__ = ["compute_score", "multiset_overlap", "format_reward", "tool_call_reward"]

_BLOCKS = {
    (True, False): r"^<think>.*?</think>\n<response>.*?</response>$",
    (False, True): r"^<think>.*?</think>\n<tool_call>\n.*?\n</tool_call>$",
    (True, True): r"^<think>.*?</think>\n<tool_call>\n.*?\n</tool_call>\n<response>.*?</response>$",
    (False, False): r"^<think>.*?</think>$",
}


def multiset_overlap(a: list, b: list) -> float:
    """|a ∩ b| / |a ∪ b| on multisets (order ignored, multiplicities kept); 1.0 for equal lists, 0.0 if one is empty."""
    if a == b:
        return 1.0
    if not a or not b:
        return 0.0
    ca, cb = Counter(a), Counter(b)
    inter = sum((ca & cb).values())
    union = len(a) + len(b) - inter
    return inter / union if union > 0 else 0.0


def format_reward(reply: str, answer: str, hi: float = 1.0, lo: float = 0.0) -> float:
    has_resp, has_tool = "<response>" in answer, "<tool_call>" in answer
    if not re.search(_BLOCKS[(has_resp, has_tool)], reply, re.DOTALL):
        return lo
    for tag, needed in (("response", has_resp), ("tool_call", has_tool)):
        if needed and (reply.count(f"<{tag}>") != 1 or reply.count(f"</{tag}>") != 1):
            return lo
    return hi


def _parse_calls(text: str) -> list:
    body = text.split("<tool_call>")[1].split("</tool_call>")[0].strip()
    return [json.loads(line) for line in body.split("\n")]


def tool_call_reward(gt_tools: list, pd_tools: list, hi: float = 3.0, lo: float = -3.0) -> float:
    if gt_tools == pd_tools:
        return hi
    score = multiset_overlap([t["name"] for t in gt_tools], [t["name"] for t in pd_tools])
    best_possible = 1.0
    used: set = set()
    for gt in gt_tools:
        params = gt["parameters"]
        best_possible += 1.0 + len(params)
        best, best_i = 0.0, -1
        for i, pd in enumerate(pd_tools):
            if i in used or pd["name"] != gt["name"]:
                continue
            got = pd["parameters"]
            s = multiset_overlap(list(params), list(got)) + sum(1.0 for k, v in params.items() if k in got and got[k] == v)
            if s > best:
                best, best_i = s, i
        if best_i >= 0:
            used.add(best_i)
            score += best
    return (hi - lo) * score / best_possible + lo


def _assistant_text(solution_str: str, experiment_name: str) -> str:
    if "llama" in experiment_name:
        return solution_str.split("<|start_header_id|>assistant<|end_header_id|>")[-1].split("<|eot_id|>")[0].strip()
    if "qwen" in experiment_name:
        return solution_str.split("<|im_start|>assistant")[-1].split("<|im_end|>")[0].strip()
    raise NotImplementedError(f"Unknown model name: {experiment_name}")


def compute_score(data_source, solution_str: str, ground_truth: str, extra_info=None, step: int = 0) -> dict:
    reply = _assistant_text(solution_str, (extra_info or {}).get("experiment_name", ""))
    fmt = format_reward(reply, ground_truth)
    acc = 0.0
    if "<tool_call>" in ground_truth:
        try:
            if "<tool_call>" not in reply or "</tool_call>" not in reply:
                raise ValueError("no tool call block")
            acc = tool_call_reward(_parse_calls(ground_truth), _parse_calls(reply))
        except Exception:  # noqa: BLE001 - malformed reply: the lowest score
            acc = -3.0
    return {"score": fmt + acc, "format_reward": fmt, "accuracy_reward": acc}
