"""Code-generation scorer: run the generated program against input/output test cases in a throw-away child process.

Ground truth: ``{"inputs": [...], "outputs": [...]}`` (or its JSON text), optionally with ``"fn_name"``. Without ``fn_name``
the program reads stdin and its stdout is compared with the expected output (whitespace-normalised, numbers compared with a
tolerance); with ``fn_name`` the function is called with the (JSON-decoded) arguments and its return value compared.
Every test runs in its own ``python -I`` subprocess with a wall-clock limit, an address-space limit and no inherited
environment, in an empty temporary directory; the child is killed by its exact PID on timeout. ``continuous=True`` scores the
fraction of the first ten tests that pass, otherwise all tests must pass.

Reference: ``verl/utils/reward_score/prime_code/__init__.py`` (APPS-style checker); the remote ``sandbox_fusion`` service of
the reference is replaced by this local sandbox when no URL is configured.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

__all__ = ["compute_score", "extract_code", "run_case"]

_RUNNER = r'''
import json, sys
src, fn_name, args = json.loads(sys.stdin.read())
g = {"__name__": "__main__"}
if fn_name is None:
    import io
    sys.stdin = io.StringIO(args)
    exec(compile(src, "<solution>", "exec"), g)
else:
    g["__name__"] = "solution"
    exec(compile(src, "<solution>", "exec"), g)
    f = g.get(fn_name)
    if f is None and "Solution" in g:
        f = getattr(g["Solution"](), fn_name)
    out = f(*args)
    sys.stdout.write("\n__RETURN__" + json.dumps(out, default=list))
'''


def extract_code(completion: str) -> str:
    """The last ```python fenced block (or any fenced block), else the completion itself."""
    if "```python" in completion:
        return completion.split("```python")[-1].split("```")[0]
    if "```" in completion:
        parts = completion.split("```")
        if len(parts) >= 3:
            return parts[-2].split("\n", 1)[-1] if parts[-2].split("\n", 1)[0].strip().isalpha() else parts[-2]
    return completion


def _limits(memory_mb: int):
    def apply():
        try:
            import resource

            resource.setrlimit(resource.RLIMIT_AS, (memory_mb << 20, memory_mb << 20))
            resource.setrlimit(resource.RLIMIT_NPROC, (64, 64))
            resource.setrlimit(resource.RLIMIT_FSIZE, (16 << 20, 16 << 20))
        except Exception:  # noqa: BLE001 - limits are best effort
            pass
        os.setsid()

    return apply


def run_case(code: str, stdin_or_args, fn_name=None, timeout: float = 5.0, memory_mb: int = 1024):
    """→ (status, output) with status in {"ok", "timeout", "error"}."""
    payload = json.dumps([code, fn_name, stdin_or_args])
    with tempfile.TemporaryDirectory(prefix="verl_b200_sandbox_") as tmp:
        proc = subprocess.Popen([sys.executable, "-I", "-c", _RUNNER], stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                cwd=tmp, env={"PATH": "/usr/bin:/bin"}, preexec_fn=_limits(memory_mb), text=True)
        try:
            out, err = proc.communicate(payload, timeout=timeout)
        except subprocess.TimeoutExpired:
            try:
                os.killpg(proc.pid, 9)           # the child is its own process group (setsid above)
            except OSError:
                proc.kill()
            proc.communicate()
            return "timeout", ""
        if proc.returncode != 0:
            return "error", err[-500:]
        return "ok", out


def _norm_tokens(s: str):
    return str(s).split()


def _same(got: str, want) -> bool:
    if isinstance(want, list) and not isinstance(want, str):
        want = "\n".join(str(x) for x in want)
    g, w = _norm_tokens(got), _norm_tokens(want)
    if g == w:
        return True
    if len(g) != len(w):
        return False
    try:
        return all(abs(float(a) - float(b)) <= 1e-6 * max(1.0, abs(float(b))) for a, b in zip(g, w))
    except ValueError:
        return False


def compute_score(completion: str, test_cases, continuous: bool = False, timeout: float = 5.0, max_tests: int = 10):
    """→ (score, per-test records). ``score`` is a bool (all tests) or, with ``continuous``, the passed fraction."""
    if not isinstance(test_cases, dict):
        try:
            test_cases = json.loads(test_cases)
        except Exception:  # noqa: BLE001
            return (0.0 if continuous else False), [{"error": "unparsable test cases"}]
    code = extract_code(str(completion))
    inputs, outputs = list(test_cases.get("inputs", [])), list(test_cases.get("outputs", []))
    fn_name = test_cases.get("fn_name")
    n = min(len(inputs), len(outputs))
    if n == 0:
        return (0.0 if continuous else False), [{"error": "no test cases"}]
    if continuous:
        n = min(n, max_tests)
    records, passed = [], 0
    for i in range(n):
        arg = inputs[i]
        if fn_name is None and isinstance(arg, list):
            arg = "\n".join(str(x) for x in arg)
        status, out = run_case(code, arg, fn_name, timeout)
        ok = False
        if status == "ok":
            if fn_name is None:
                ok = _same(out, outputs[i])
            else:
                ret = out.rsplit("\n__RETURN__", 1)
                if len(ret) == 2:
                    try:
                        got = json.loads(ret[1])
                        want = outputs[i]
                        ok = got == want or (isinstance(want, list) and len(want) == 1 and got == want[0])
                    except json.JSONDecodeError:
                        ok = False
        records.append({"test": i, "status": status, "passed": ok})
        passed += ok
        if not ok and not continuous:
            return False, records
    return (passed / n if continuous else passed == n), records
