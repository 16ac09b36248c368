"""MATH-style: compare the last ``\\boxed{...}`` of the response with the normalised ground truth."""

import re


def last_boxed_only_string(s: str):
    idx = s.rfind("\\boxed")
    if idx < 0:
        idx = s.rfind("\\fbox")
        if idx < 0:
            return None
    depth, end = 0, None
    for i in range(idx, len(s)):
        if s[i] == "{":
            depth += 1
        elif s[i] == "}":
            depth -= 1
            if depth == 0:
                end = i
                break
    return s[idx : end + 1] if end is not None else None


def remove_boxed(s: str) -> str:
    if s.startswith("\\boxed "):
        return s[len("\\boxed "):]
    left = "\\boxed{"
    return s[len(left):-1] if s.startswith(left) and s.endswith("}") else s


def normalize(ans: str) -> str:
    ans = ans.strip().replace("\\!", "").replace("\\,", "").replace(" ", "").replace("dfrac", "frac").replace("tfrac", "frac")
    ans = ans.replace("\\left", "").replace("\\right", "").replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "").replace("$", "")
    ans = re.sub(r"\\text\{([^}]*)\}", r"\1", ans)
    if ans.endswith("."):
        ans = ans[:-1]
    if ans.startswith("0.") is False and ans.startswith("."):
        ans = "0" + ans
    return ans


def compute_score(solution_str: str, ground_truth: str) -> float:
    try:
        boxed = last_boxed_only_string(solution_str)
        if boxed is None:
            return 0.0
        return 1.0 if normalize(remove_boxed(boxed)) == normalize(str(ground_truth)) else 0.0
    except Exception:
        return 0.0


def is_equiv(a: str, b: str) -> bool:
    """Answers are equivalent when their normalised forms match as text (or as numbers when both parse)."""
    na, nb = normalize(a), normalize(b)
    if na == nb:
        return True
    try:
        return abs(float(na) - float(nb)) < 1e-9
    except ValueError:
        return False
