"""HellaSwag → training parquet for a model-based (or exact-match) reward (reference: examples/data_preprocess/hellaswag.py): the
prompt is the context, the ground truth the gold ending; the candidate endings travel in `extra_info`."""

import re

from _common import build, parser, row

DATA_SOURCE = "Rowan/hellaswag"


def clean(text: str) -> str:
    text = text.strip().replace(" [title]", ". ")
    return re.sub(r"\[.*?\]", "", text).replace("  ", " ")


def to_row(ex, idx, split):
    if ex.get("label", "") in ("", None):
        return None                                     # the public test split carries no labels
    ctx = clean(f"{ex['activity_label']}: {ex['ctx_a']} {ex['ctx_b'].capitalize()}")
    endings = [clean(e) for e in ex["endings"]]
    return row(DATA_SOURCE, [{"role": "user", "content": ctx}], "nlp", endings[int(ex["label"])], split, idx, style="model", endings=endings)


if __name__ == "__main__":
    build(parser("~/data/hellaswag", __doc__).parse_args(), DATA_SOURCE, to_row, splits=("train", "test"), split_alias={"test": "validation"})
