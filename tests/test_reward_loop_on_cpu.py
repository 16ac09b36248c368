"""Reward-loop managers and the extra rule-based scorers."""

import asyncio
import time

import pytest

import torch

from verl_b200.experimental.reward_loop import RewardLoopManager, get_reward_loop_manager_cls
from verl_b200.protocol import DataProto
from verl_b200.utils.config import Config
from verl_b200.utils.reward_score import default_compute_score
from verl_b200.utils.tokenizer import ByteChatTokenizer


def test_scorers():
    assert default_compute_score("math_dapo", "blah blah\nAnswer: $\\boxed{42}$", "42")["score"] == 1.0
    assert default_compute_score("aime2024", "Answer: 7", "8")["score"] == -1.0
    assert default_compute_score("searchR1_nq", "<answer>The Eiffel Tower</answer>", {"target": ["eiffel tower"]}) == 1.0
    s = default_compute_score("geo3k", "<think>x</think> so \\boxed{12}", "12")
    assert abs(s - 1.0) < 1e-9 and default_compute_score("geo3k", "\\boxed{12}", "12") == 0.9


def _batch(tok, texts, R=24):
    ids = torch.full((len(texts), 4 + R), tok.pad_token_id)
    att = torch.zeros(len(texts), 4 + R, dtype=torch.int64)
    att[:, :4] = 1
    for i, t in enumerate(texts):
        e = tok.encode(t)
        ids[i, 4: 4 + len(e)] = torch.tensor(e)
        att[i, 4: 4 + len(e)] = 1
    return DataProto.from_dict(tensors={"input_ids": ids, "attention_mask": att, "responses": ids[:, 4:]},
                               non_tensors={"data_source": ["gsm8k"] * len(texts), "reward_model": [{"ground_truth": "5"}] * len(texts)})


def test_reward_loop_manager_scores_at_last_token():
    tok = ByteChatTokenizer()
    texts = ["so #### 5", "hmm #### 6", "#### 5"]
    mgr = RewardLoopManager(Config({"reward": {"reward_manager": "naive"}}), tok, num_workers=2)
    out = mgr.compute_rm_score(_batch(tok, texts))
    sc = out.batch["rm_scores"]
    assert sc.sum(-1).tolist() == [1.0, 0.0, 1.0] and sc[0, len(texts[0]) - 1] == 1.0 and sc[2, len(texts[2]) - 1] == 1.0
    assert out.non_tensor_batch["acc"].tolist() == [1.0, 0.0, 1.0]
    mgr.shutdown()


def test_dapo_overlong_gdpo_components_and_rate_limit():
    tok = ByteChatTokenizer()
    cfg = Config({"data": {"max_response_length": 20}, "reward": {"reward_kwargs": {"overlong_buffer_cfg": {"enable": True, "len": 10, "penalty_factor": 1.0, "log": True},
                                                                                     "max_concurrent": 2, "max_rpm": 0, "timeout": 0.05}}})
    dapo = get_reward_loop_manager_cls("dapo")(cfg, tok, lambda **kw: 1.0)
    r = asyncio.run(dapo.run_single({"response_str": "x", "valid_response_length": 15}))
    assert abs(r["reward_score"] - 0.5) < 1e-9 and r["reward_extra_info"]["overlong"]
    gdpo = get_reward_loop_manager_cls("gdpo")(cfg, tok, lambda **kw: {"components": {"correct": 1.0, "format": 0.25}})
    r = asyncio.run(gdpo.run_single({"response_str": "x", "valid_response_length": 1}))
    assert r["reward_score"] == 1.25 and r["reward_extra_info"]["reward_components"] == {"correct": 1.0, "format": 0.25}

    running, peak = [0], [0]

    async def slow(**kw):
        running[0] += 1
        peak[0] = max(peak[0], running[0])
        await asyncio.sleep(0.01 if kw["solution_str"] != "slow" else 1.0)
        running[0] -= 1
        return 1.0

    lim = get_reward_loop_manager_cls("limited")(cfg, tok, slow)

    async def go():
        return await asyncio.gather(*[lim.run_single({"response_str": "slow" if i == 0 else "ok", "valid_response_length": 1}) for i in range(6)])

    res = asyncio.run(go())
    assert peak[0] <= 2 and res[0]["reward_extra_info"].get("timeout") and res[1]["reward_score"] == 1.0


def test_prime_math_and_code_scorers():
    from verl_b200.utils.reward_score import default_compute_score, prime_code, prime_math

    assert prime_math.compute_score("Step 2: so \\boxed{\\frac{1}{2}}", "0.5")[:2] == (True, True)
    assert prime_math.compute_score("The answer is 50%", "0.5")[0] and prime_math.compute_score("\\boxed{2\\pi}", "6.2832")[0]
    assert prime_math.compute_score("\\boxed{(1, 2.0)}", "(1,2)")[0] and not prime_math.compute_score("\\boxed{(1, 3)}", "(1,2)")[0]
    assert not prime_math.compute_score("\\boxed{7}", "8")[0]
    assert default_compute_score("numina_cn_k12", "\\boxed{x=3}", "3") == 1.0

    tests = {"inputs": ["1 2\n", "10 20\n", "5 5\n"], "outputs": ["3\n", "30\n", "10\n"]}
    good = "Here:\n```python\na, b = map(int, input().split())\nprint(a + b)\n```"
    half = "```python\na, b = map(int, input().split())\nprint(a + b if a < 10 else 0)\n```"
    assert prime_code.compute_score(good, tests)[0] is True
    score, recs = prime_code.compute_score(half, tests, continuous=True)
    assert abs(score - 2 / 3) < 1e-9 and [r["passed"] for r in recs] == [True, False, True]
    slow = "```python\nwhile True:\n    pass\n```"
    ok, recs = prime_code.compute_score(slow, tests, timeout=1.0)
    assert ok is False and recs[0]["status"] == "timeout"
    boom = "```python\nraise SystemExit(3)\n```"
    assert prime_code.compute_score(boom, tests)[1][0]["status"] == "error"
    fn = {"fn_name": "add", "inputs": [[1, 2], [3, 4]], "outputs": [3, [7]]}
    assert prime_code.compute_score("```python\ndef add(a, b):\n    return a + b\n```", fn)[0] is True
    assert default_compute_score("apps", good, tests) == 1.0


def test_sandbox_fusion_client_against_a_local_service():
    """The remote code scorer posts every test case to a sandbox service; here a stand-in service on 127.0.0.1 runs the posted
    program with the local sandbox and answers in the service's JSON form. One request fails with 503 first (retried)."""
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    from verl_b200.utils.reward_score import default_compute_score, sandbox_fusion
    from verl_b200.utils.reward_score.prime_code import run_case

    state = {"calls": 0, "failed_once": False}

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            req = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            state["calls"] += 1
            if not state["failed_once"]:
                state["failed_once"] = True
                self.send_response(503)
                self.end_headers()
                return
            status, out = run_case(req["code"], req["stdin"], None, timeout=float(req["run_timeout"]))
            body = {"status": "Success" if status == "ok" else "Failed",
                    "run_result": {"status": "Finished" if status != "timeout" else "TimeLimitExceeded", "stdout": out if status == "ok" else "",
                                   "stderr": "" if status == "ok" else out, "return_code": 0 if status == "ok" else 1}}
            data = json.dumps(body).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    srv = ThreadingHTTPServer(("127.0.0.1", 0), Handler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{srv.server_address[1]}/run_code"
    try:
        tests = {"inputs": ["1 2\n", "5 7\n", "10 -3\n"], "outputs": ["3\n", "12\n", "7\n"]}
        good = "```python\na, b = map(int, input().split())\nprint(a + b)\n```"
        half = "```python\na, b = map(int, input().split())\nprint(a + b if a < 6 else 0)\n```"
        score, recs = sandbox_fusion.compute_score(url, None, 512, good, tests)
        assert score == 1.0 and all(r["passed"] for r in recs) and state["calls"] == 4          # one 503 was retried
        score, _ = sandbox_fusion.compute_score(url, threading.Semaphore(2), 512, half, tests, continuous=True)
        assert abs(score - 2 / 3) < 1e-6
        fn_tests = {"fn_name": "add", "inputs": [[1, 2], [3, 4]], "outputs": [3, 7]}
        assert sandbox_fusion.compute_score(url, None, 512, "def add(a, b):\n    return a + b\n", fn_tests)[0] == 1.0
        assert sandbox_fusion.compute_score(url, None, 512, "def add(a, b):\n    return a - b\n", fn_tests)[0] == 0.0
        # dispatch by data source with the service configured
        assert default_compute_score("codecontests", good, json.dumps(tests), sandbox_fusion_url=url) == 1.0
    finally:
        srv.shutdown()
    # an unreachable service scores 0 instead of raising
    score, recs = sandbox_fusion.compute_score("http://127.0.0.1:9/run_code", None, 512, good, tests, timeout=0.5)
    assert score == 0.0 and recs[0]["status"] == "sandbox_error"


def _slow_or_fast(task, completion, reference, extra):
    import time

    if completion == "hang":
        time.sleep(30)
    if completion == "boom":
        raise RuntimeError("checker crashed")
    return (1.0, "details") if completion == reference else {"score": 0.25}


def _fake_verify(gold, out):
    return 1.0 if gold == "\\boxed{" + out + "}" else 0.0


def test_prime_manager_rlla_and_math_verify():
    import numpy as np
    import torch

    from verl_b200.protocol import DataProto
    from verl_b200.utils.reward_score import default_compute_score, math_verify, rlla
    from verl_b200.workers.reward_manager import get_reward_manager_cls
    from verl_b200.workers.reward_manager.prime import run_reward_scoring

    # process-pool scoring: tuple / dict / failing / hanging checkers
    s = run_reward_scoring(_slow_or_fast, ["a", "b", "boom", "hang"], ["a", "x", "y", "z"], ["t"] * 4, None, num_processes=4, timeout=2.0)
    assert s == [1.0, 0.25, 0.0, 0.0]
    mgr = get_reward_manager_cls("prime")(tokenizer=None, compute_score=_slow_or_fast, num_processes=2, timeout=5.0)
    data = DataProto.from_dict(tensors={"prompts": torch.zeros(2, 3, dtype=torch.long), "responses": torch.tensor([[7, 8, 0], [9, 0, 0]]),
                                        "attention_mask": torch.tensor([[1, 1, 1, 1, 1, 0], [0, 1, 1, 1, 0, 0]])},
                               non_tensors={"data_source": np.array(["t", "t"], dtype=object),
                                            "reward_model": np.array([{"ground_truth": "7 8"}, {"ground_truth": "nope"}], dtype=object)})
    out = mgr(data, return_dict=True)
    assert out["reward_tensor"].tolist() == [[0.0, 1.0, 0.0], [0.25, 0.0, 0.0]] and data.batch["acc"].tolist() == [1.0, 0.25]

    # tool-use reward: exact call = +3 and format +1; a wrong parameter value lowers the correctness term; malformed = -3
    gt = '<think>plan</think>\n<tool_call>\n{"name": "search", "parameters": {"q": "b200", "k": 3}}\n</tool_call>'
    wrap = lambda body: "<|im_start|>assistant" + body + "<|im_end|>"      # noqa: E731
    info = {"experiment_name": "qwen-test"}
    full = rlla.compute_score("rlla", wrap(gt), gt, info)
    assert full == {"score": 4.0, "format_reward": 1.0, "accuracy_reward": 3.0}
    off = rlla.compute_score("rlla", wrap(gt.replace('"k": 3', '"k": 5')), gt, info)
    assert off["format_reward"] == 1.0 and -3.0 < off["accuracy_reward"] < 3.0
    bad = rlla.compute_score("rlla", wrap("<think>x</think>\nno call here"), gt, info)
    assert bad == {"score": -3.0, "format_reward": 0.0, "accuracy_reward": -3.0}
    assert rlla.multiset_overlap(["a", "a", "b"], ["a", "b", "b"]) == 0.5
    assert default_compute_score("rlla", wrap(gt), gt, info)["score"] == 4.0
    with pytest.raises(NotImplementedError):
        rlla.compute_score("rlla", "x", gt, {"experiment_name": "other"})

    # math_verify: same pool / time-out path with a stand-in verifier; without the package the scorer refuses to run
    assert math_verify.compute_score("42", "42", _verify_fn=_fake_verify) == 1.0 and math_verify.compute_score("41", "42", _verify_fn=_fake_verify) == 0.0
    if not math_verify.available():
        with pytest.raises(ImportError):
            math_verify.compute_score("42", "42")


def test_reward_model_manager_serves_replicas_behind_a_router():
    """Two in-process judge replicas behind the router: requests spread over both, a repeated request id stays on its replica,
    answers equal the engine's own, and the `remote` reward-loop manager scores through the router client."""
    import asyncio
    import json
    import urllib.request

    import torch

    from verl_b200.experimental.reward_loop import RewardLoopManager, RewardModelManager
    from verl_b200.models.config import PRESETS
    from verl_b200.models.transformer import DecoderLM
    from verl_b200.utils.tokenizer import ByteChatTokenizer
    from verl_b200.workers.rollout.engine import InferenceEngine, SamplingParams

    model = DecoderLM(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=3)
    engines = [InferenceEngine(model, max_num_seqs=8, max_model_len=128, num_blocks=32) for _ in range(2)]
    tok = ByteChatTokenizer()
    mgr = RewardModelManager({"rollout": {"tensor_model_parallel_size": 1, "free_cache_engine": False}}, engines=engines, tokenizer=tok)
    try:
        assert len(mgr.server_addresses) == 2 and json.load(urllib.request.urlopen(f"http://{mgr.get_router_address()}/health"))["workers"] == 2
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(10, 250, (12,), generator=g).tolist() for _ in range(8)]
        sp = SamplingParams(temperature=0.0, max_tokens=6)
        want = engines[0].generate(prompts, sp)
        client = mgr.client()

        async def go():
            outs = await asyncio.gather(*[client.generate(f"req-{i}", p, sp) for i, p in enumerate(prompts)])
            again = await client.generate("req-0", prompts[0], sp)
            await client.close()
            return outs, again

        outs, again = asyncio.run(go())
        for o, w in zip(outs, want):
            assert o.token_ids == w.token_ids
        assert again.token_ids == want[0].token_ids
        served = {w["url"]: w["served"] for w in json.load(urllib.request.urlopen(f"http://{mgr.get_router_address()}/workers"))["workers"]}
        assert sum(served.values()) == 9 and min(served.values()) >= 3          # both replicas took a share
        first = mgr.router.sticky["req-0"]
        assert mgr.router.sticky["req-0"] == first and len(mgr.router.sticky) == 8
        # the remote reward-loop manager scores a sample through the router: the judge's text is parsed for a number
        loop_mgr = RewardLoopManager({"reward": {"reward_manager": "remote", "reward_kwargs": {"judge_max_tokens": 4}}}, tok, None, num_workers=2,
                                     manager_name="remote", rm_client=mgr.client())
        s = asyncio.run(loop_mgr.workers[0].compute_score({"prompt_ids": prompts[0], "response_ids": prompts[1][:5]}))
        assert isinstance(s["reward_score"], float) and "rm_score" in s["reward_extra_info"]
        loop_mgr.shutdown()
        mgr.sleep()
        assert all(e.cache is None for e in engines)
        mgr.wake_up()
    finally:
        mgr.shutdown()
