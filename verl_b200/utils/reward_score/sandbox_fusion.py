"""Code scorer that runs the test cases on a remote sandbox service (``POST <url>`` with ``{"code", "stdin", "language",
"run_timeout", "memory_limit_MB"}``; answer ``{"status": "Success" | ..., "run_result": {"status", "stdout", "stderr",
"return_code"}}``). Test cases have the ``{"inputs": [...], "outputs": [...], "fn_name"?}`` form of the local scorer
(:mod:`verl_b200.utils.reward_score.prime_code`); cases are posted concurrently (bounded by ``max_concurrency`` or a
caller-provided semaphore), transient HTTP errors (429 / 5xx / connection) are retried with back-off.

Reference: ``verl/utils/reward_score/sandbox_fusion/{__init__,utils}.py`` (``compute_score(sandbox_fusion_url,
concurrent_semaphore, memory_limit_mb, completion, test_cases, continuous)``).
"""

from __future__ import annotations

import json
import threading
import time
import urllib.error
import urllib.request
from concurrent.futures import ThreadPoolExecutor

from .prime_code import _same, extract_code

__all__ = ["compute_score", "call_sandbox"]

_FN_WRAPPER = '''
import json, sys
{code}
_args = json.loads(sys.stdin.read())
_f = globals().get({fn!r})
if _f is None and "Solution" in globals():
    _f = getattr(Solution(), {fn!r})
print("__RETURN__" + json.dumps(_f(*_args), default=list))
'''


def call_sandbox(url: str, code: str, stdin: str, timeout: float = 10.0, memory_limit_mb: int = 1024, language: str = "python",
                 retries: int = 3) -> dict:
    """One ``run_code`` request → the decoded JSON answer, or ``{"status": "SandboxError", "message": ...}``."""
    body = json.dumps({"code": code, "stdin": stdin, "language": language, "compile_timeout": timeout, "run_timeout": timeout,
                       "memory_limit_MB": memory_limit_mb}).encode()
    err = "no attempt made"
    for attempt in range(retries):
        try:
            req = urllib.request.Request(url, data=body, headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=timeout + 10) as resp:
                return json.loads(resp.read().decode())
        except urllib.error.HTTPError as e:
            err = f"HTTP {e.code}"
            if e.code not in (429, 500, 502, 503, 504):
                break
        except Exception as e:  # noqa: BLE001 - connection refused / reset / timeout: retry
            err = f"{type(e).__name__}: {e}"
        time.sleep(0.2 * (2 ** attempt))
    return {"status": "SandboxError", "message": err}


def _check_case(url, code, fn_name, arg, want, timeout, memory_limit_mb, sem) -> dict:
    if fn_name is None:
        program, stdin = code, "\n".join(str(x) for x in arg) if isinstance(arg, list) else str(arg)
    else:
        program, stdin = _FN_WRAPPER.format(code=code, fn=fn_name), json.dumps(arg)
    with sem:
        ans = call_sandbox(url, program, stdin, timeout, memory_limit_mb)
    run = ans.get("run_result") or {}
    if ans.get("status") != "Success" or run.get("return_code", 1) != 0:
        status = "timeout" if "TimeLimit" in str(run.get("status", "")) else ("sandbox_error" if ans.get("status") == "SandboxError" else "error")
        return {"status": status, "passed": False}
    out = run.get("stdout", "")
    if fn_name is None:
        return {"status": "ok", "passed": _same(out, want)}
    ret = out.rsplit("__RETURN__", 1)
    try:
        got = json.loads(ret[1]) if len(ret) == 2 else None
    except json.JSONDecodeError:
        return {"status": "ok", "passed": False}
    return {"status": "ok", "passed": got == want or (isinstance(want, list) and len(want) == 1 and got == want[0])}


def compute_score(sandbox_fusion_url: str, concurrent_semaphore, memory_limit_mb: int, completion: str, test_cases, continuous: bool = False,
                  timeout: float = 10.0, max_tests: int = 10, max_concurrency: int = 8):
    """→ (score, per-test records); ``score`` is the passed fraction (``continuous``) or 1.0/0.0 for all-pass."""
    if not isinstance(test_cases, dict):
        try:
            test_cases = json.loads(test_cases)
        except Exception:  # noqa: BLE001
            return 0.0, [{"error": "unparsable test cases"}]
    inputs, outputs = list(test_cases.get("inputs", [])), list(test_cases.get("outputs", []))
    n = min(len(inputs), len(outputs))
    if n == 0:
        return 0.0, [{"error": "no test cases"}]
    if continuous:
        n = min(n, max_tests)
    code, fn_name = extract_code(str(completion)), test_cases.get("fn_name")
    sem = concurrent_semaphore if concurrent_semaphore is not None else threading.Semaphore(max_concurrency)
    with ThreadPoolExecutor(max_workers=min(n, max_concurrency)) as ex:
        records = list(ex.map(lambda i: _check_case(sandbox_fusion_url, code, fn_name, inputs[i], outputs[i], timeout, memory_limit_mb, sem), range(n)))
    passed = sum(r["passed"] for r in records)
    return (passed / n if continuous else float(passed == n)), records
