"""Exact-match QA scoring on the text inside the last ``<answer>…</answer>`` (reference:
``verl/utils/reward_score/search_r1_like_qa_em.py``)."""

from __future__ import annotations

import re
import string


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def extract_solution(text: str):
    m = re.findall(r"<answer>(.*?)</answer>", text, re.DOTALL)
    return m[-1].strip() if len(m) >= 1 else None


def compute_score(solution_str: str, ground_truth, format_score: float = 0.0, score: float = 1.0, **kwargs) -> float:
    ans = extract_solution(solution_str)
    if ans is None:
        return 0.0
    targets = ground_truth["target"] if isinstance(ground_truth, dict) else ground_truth
    targets = [targets] if isinstance(targets, str) else list(targets)
    return score if any(normalize_answer(ans) == normalize_answer(t) for t in targets) else format_score
