"""GSM8K → training parquet (reference: examples/data_preprocess/gsm8k.py). `python examples/data_preprocess/gsm8k.py --local_dataset_path raw/gsm8k`"""

import re

from _common import build, parser, row

DATA_SOURCE = "openai/gsm8k"
INSTRUCTION = 'Let\'s think step by step and output the final answer after "####".'


def extract_solution(answer: str) -> str:
    m = re.search(r"#### (\-?[0-9\.\,]+)", answer)
    assert m is not None, f"no '#### <number>' in {answer[-80:]!r}"
    return m.group(1).replace(",", "")


def to_row(ex, idx, split):
    q, a = ex["question"], ex["answer"]
    return row(DATA_SOURCE, [{"role": "user", "content": f"{q} {INSTRUCTION}"}], "math", extract_solution(a), split, idx, answer=a, question=q)


if __name__ == "__main__":
    build(parser("~/data/gsm8k", __doc__).parse_args(), DATA_SOURCE, to_row, hub_config="main")
