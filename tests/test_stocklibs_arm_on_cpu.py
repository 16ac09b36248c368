"""The stock-library baseline arm of bench.py: its training half (transformers + torch AdamW, packed micro-batches, GRPO
loss) runs on CPU against a stand-in rollout engine, so that a GPU run only has to prove the vLLM half."""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))


class _Completion:
    def __init__(self, ids):
        self.token_ids = ids


class _Out:
    def __init__(self, outs):
        self.outputs = outs


class FakeLLM:
    """Uniform random tokens, n completions per prompt; records the calls the arm makes."""

    def __init__(self, n, R):
        self.n, self.R, self.calls = n, R, []

    def sleep(self, level=1):
        self.calls.append("sleep")

    def wake_up(self):
        self.calls.append("wake")

    def collective_rpc(self, fn):
        self.calls.append("sync")

    def generate(self, prompts, sp, use_tqdm=False):
        g = torch.Generator().manual_seed(len(self.calls))
        self.calls.append("gen")
        return [_Out([_Completion(torch.randint(10, 2000, (self.R,), generator=g).tolist()) for _ in range(self.n)]) for _ in prompts]


def test_training_half_runs_and_reports(capsys):
    import stocklibs_grpo

    args = argparse.Namespace(model="tiny-qwen2", prompts_per_gpu=4, mini_prompts_per_gpu=2, n=2, min_prompt=8, max_prompt=16, response_length=8,
                              token_budget=64, steps=1, warmup=1, time_limit=0.0, verbose=False, vllm_util=0.3)
    llm = FakeLLM(2, 8)
    out = stocklibs_grpo.run(args, llm=llm, sampling=None)
    assert out["impl"] == "stocklibs" and out["steps"] == 1 and out["warmup"] == 1 and out["value"] > 0
    assert out["tokens_per_step"] == sum(out_len for out_len in [out["tokens_per_step"]])
    assert set(out["step_breakdown_s"]) == {"gen", "old_log_prob", "ref", "update_actor", "step"}
    # per step: wake, weight push, generate, sleep (after the initial sleep)
    assert llm.calls == ["sleep"] + ["wake", "sync", "gen", "sleep"] * 2


def test_micro_batches_respect_the_token_budget():
    import stocklibs_grpo

    lens = [5, 9, 3, 7, 8, 2]
    mbs = stocklibs_grpo._micro_batches(lens, 12)
    assert sorted(i for mb in mbs for i in mb) == list(range(6))
    assert all(sum(lens[i] for i in mb) <= 12 for mb in mbs)
