"""Anthropic HH-RLHF (helpful-base style rows with `prompt`, `response`, `chosen`, `rejected`) → prompt-only parquet for PPO with a reward
model (reference: examples/data_preprocess/full_hh_rlhf.py, its `rl` split)."""

from _common import build, parser, row

DATA_SOURCE = "Dahoas/full-hh-rlhf"


def to_row(ex, idx, split):
    return row(DATA_SOURCE, [{"role": "user", "content": ex["prompt"]}], "alignment", ex.get("response", ex.get("chosen", "")), split, idx, style="model")


if __name__ == "__main__":
    build(parser("~/data/full_hh_rlhf/rl", __doc__).parse_args(), DATA_SOURCE, to_row, splits=("train",))
