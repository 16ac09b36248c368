"""MATH (lighteval mirror) → training parquet (reference: examples/data_preprocess/math_dataset.py); the ground truth is the content of
the last \\boxed{} of the worked solution."""

from _common import build, parser, row

from verl_b200.utils.reward_score.math_reward import last_boxed_only_string, remove_boxed

DATA_SOURCE = "DigitalLearningGmbH/MATH-lighteval"
INSTRUCTION = "Let's think step by step and output the final answer within \\boxed{}."


def to_row(ex, idx, split):
    boxed = last_boxed_only_string(ex["solution"])
    if boxed is None:
        return None
    return row(DATA_SOURCE, [{"role": "user", "content": f"{ex['problem']} {INSTRUCTION}"}], "math", remove_boxed(boxed), split, idx)


if __name__ == "__main__":
    build(parser("~/data/math", __doc__).parse_args(), DATA_SOURCE, to_row)
