"""Geometry3K (vision-language) → training parquet with an `images` column (reference: examples/data_preprocess/geo3k.py): the prompt
marks the picture with `<image>`, which the dataset expands to the model's placeholder tokens."""

from _common import build, parser, row

DATA_SOURCE = "hiyouga/geometry3k"
INSTRUCTION = (r"You FIRST think about the reasoning process as an internal monologue and then provide the final answer. "
               r"The reasoning process MUST BE enclosed within <think> </think> tags. The final answer MUST BE put in \boxed{}.")


def to_row(ex, idx, split):
    problem = ex["problem"]
    if "<image>" not in problem:
        problem = "<image>" + problem
    return row(DATA_SOURCE, [{"role": "user", "content": f"{problem} {INSTRUCTION}"}], "math", ex["answer"], split, idx, answer=ex["answer"],
               question=ex["problem"], images=ex["images"])


if __name__ == "__main__":
    build(parser("~/data/geo3k", __doc__).parse_args(), DATA_SOURCE, to_row)
