"""Math grader for the NuminaMath-style sources: extract the final answer, then try string normalisation, numeric
comparison (fractions, percentages, pi as a symbol or 3.14), tuples/intervals element-wise and finally a symbolic difference
when sympy is importable. Returns ``(is_correct, format_ok, extracted_answer)`` like the reference
(``verl/utils/reward_score/prime_math/__init__.py:389-411``)."""

from __future__ import annotations

import math
import re
from fractions import Fraction

from .math_reward import last_boxed_only_string, normalize, remove_boxed

__all__ = ["compute_score", "match_answer", "math_equal"]


def match_answer(response: str):
    """→ (found, answer): the last boxed expression, else what follows 'answer is' / 'Answer:' on the last such line."""
    boxed = last_boxed_only_string(response)
    if boxed is not None:
        return True, remove_boxed(boxed)
    m = re.findall(r"(?:answer is|Answer:|answer:)\s*([^\n]+)", response)
    if m:
        return True, m[-1].strip().rstrip(".")
    return False, response.strip().split("\n")[-1]


def _to_number(s: str, pi: float = math.pi):
    s = normalize(s).replace("\\%", "%").replace(",", "")
    pct = s.endswith("%")
    if pct:
        s = s[:-1]
    m = re.fullmatch(r"(-?)\\frac\{(-?[\d.]+)\}\{(-?[\d.]+)\}", s)
    if m:
        v = float(Fraction(m.group(2)) / Fraction(m.group(3))) * (-1 if m.group(1) else 1)
    else:
        m = re.fullmatch(r"(-?[\d.]*)\\pi", s)
        if m:
            v = (float(m.group(1)) if m.group(1) not in ("", "-") else (-1.0 if m.group(1) == "-" else 1.0)) * pi
        else:
            if "/" in s and re.fullmatch(r"-?[\d.]+/-?[\d.]+", s):
                a, b = s.split("/")
                v = float(a) / float(b)
            else:
                v = float(s)
    return v / 100.0 if pct else v


def _split_top(s: str):
    parts, depth, cur = [], 0, ""
    for ch in s:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    parts.append(cur)
    return parts


def math_equal(pred: str, ref: str, pi: float = math.pi, rel_tol: float = 1e-4) -> bool:
    a, b = normalize(str(pred)), normalize(str(ref))
    if a == b:
        return True
    try:
        x, y = _to_number(a, pi), _to_number(b, pi)
        return math.isclose(x, y, rel_tol=rel_tol, abs_tol=1e-9) or math.isclose(x * 100, y, rel_tol=rel_tol) or math.isclose(x, y * 100, rel_tol=rel_tol)
    except (ValueError, ZeroDivisionError):
        pass
    if len(a) > 1 and len(b) > 1 and a[0] in "([" and b[0] in "([" and a[-1] in ")]" and b[-1] in ")]":
        if (a[0], a[-1]) != (b[0], b[-1]):
            return False
        pa, pb = _split_top(a[1:-1]), _split_top(b[1:-1])
        return len(pa) == len(pb) and all(math_equal(u, v, pi, rel_tol) for u, v in zip(pa, pb))
    if "=" in a and "=" not in b:
        return math_equal(a.split("=")[-1], b, pi, rel_tol)
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr

        def conv(t):
            t = t.replace("^", "**").replace("\\cdot", "*").replace("\\times", "*").replace("\\pi", "pi")
            t = re.sub(r"\\frac\{([^{}]+)\}\{([^{}]+)\}", r"((\1)/(\2))", t)
            t = re.sub(r"\\sqrt\{([^{}]+)\}", r"sqrt(\1)", t)
            return parse_expr(t.replace("{", "(").replace("}", ")"))

        return bool(sympy.simplify(conv(a) - conv(b)) == 0)
    except Exception:  # noqa: BLE001 - unparsable: not equal
        return False


def compute_score(model_output: str, ground_truth: str):
    model_output, ground_truth = str(model_output), str(ground_truth)
    found, extracted = match_answer(model_output)
    format_ok = found and "\\box" in model_output
    try:
        ok = math_equal(extracted, ground_truth) or (("\\pi" in extracted or "\\pi" in ground_truth) and math_equal(extracted, ground_truth, pi=3.14))
    except Exception:  # noqa: BLE001
        ok = False
    return ok, format_ok, extracted
