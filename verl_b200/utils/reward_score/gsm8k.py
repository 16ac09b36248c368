"""GSM8K: the final answer follows ``####``; strict (that format) or flexible (last number) extraction."""

import re

_STRICT = re.compile(r"#### (\-?[0-9\.\,]+)")
_FLEX = re.compile(r"(\-?[0-9\.\,]+)")


def extract_solution(solution_str: str, method: str = "strict"):
    solution_str = solution_str[-300:]
    if method == "strict":
        found = _STRICT.findall(solution_str)
        return found[-1].replace(",", "").replace("$", "") if found else None
    found = [x for x in _FLEX.findall(solution_str) if x not in ("", ".")]
    return found[-1] if found else None


def compute_score(solution_str: str, ground_truth: str, method: str = "strict", format_score: float = 0.0, score: float = 1.0) -> float:
    ans = extract_solution(solution_str, method)
    if ans is None:
        return 0.0
    return score if ans == str(ground_truth) else format_score
