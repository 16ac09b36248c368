"""GSM8K for multi-turn rollouts with the `calc_gsm8k_reward` tool (reference: examples/data_preprocess/gsm8k_multiturn_w_tool.py):
a system turn that tells the policy to call the tool, and per-row tool construction arguments in `extra_info.tools_kwargs`."""

from _common import build, parser, row
from gsm8k import DATA_SOURCE, INSTRUCTION, extract_solution

SYSTEM = ("You are a math expert. You are given a question and you need to solve it step by step. Reasoning step by step before any tool call. "
          "You should use the `calc_gsm8k_reward` tool after step by step solving the question, before generate final answer at least once "
          "and refine your answer if necessary. Put your final answer in the format of `#### <answer>`.")


def to_row(ex, idx, split):
    q, a = ex["question"], ex["answer"]
    sol = extract_solution(a)
    msgs = [{"role": "system", "content": SYSTEM}, {"role": "user", "content": f"{q} {INSTRUCTION}"}]
    return row(DATA_SOURCE, msgs, "math", sol, split, idx, answer=a, question=q, need_tools_kwargs=True,
               tools_kwargs={"calc_gsm8k_reward": {"create_kwargs": {"ground_truth": sol}}})


if __name__ == "__main__":
    build(parser("~/data/gsm8k_multiturn_w_tool", __doc__).parse_args(), DATA_SOURCE, to_row, hub_config="main")
