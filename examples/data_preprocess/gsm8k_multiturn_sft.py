"""GSM8K as two-turn conversations for the multi-turn SFT trainer (reference: examples/data_preprocess/gsm8k_multiturn_sft.py):
rows carry a `messages` column (user question, assistant solution)."""

import os

import pandas as pd
from _common import load_split, parser
from gsm8k import DATA_SOURCE, INSTRUCTION

if __name__ == "__main__":
    args = parser("~/data/gsm8k_sft", __doc__).parse_args()
    out = os.path.expanduser(args.local_dir or args.local_save_dir)
    os.makedirs(out, exist_ok=True)
    for split in ("train", "test"):
        raw = load_split(args.local_dataset_path, DATA_SOURCE, split, "main")
        raw = raw[: args.max_rows] if args.max_rows else raw
        rows = [{"messages": [{"role": "user", "content": f"{ex['question']} {INSTRUCTION}"}, {"role": "assistant", "content": ex["answer"]}],
                 "data_source": DATA_SOURCE, "extra_info": {"split": split, "index": i}} for i, ex in enumerate(raw)]
        pd.DataFrame(rows).to_parquet(os.path.join(out, f"{split}.parquet"))
        print(f"{split}: {len(rows)} conversations")
