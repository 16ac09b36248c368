"""Search-R1 style question answering (NQ / HotpotQA rows with `question` and `golden_answers`) for multi-turn rollouts with a search tool
(reference: examples/data_preprocess/preprocess_search_r1_dataset.py): exact-match reward against any golden answer."""

from _common import build, parser, row

DATA_SOURCE = "searchR1_nq"
SYSTEM = ("Answer the given question. You must conduct reasoning inside <think> and </think> first every time you get new information. "
          "After reasoning, if you find you lack some knowledge, you can call the search tool and it will return the top results. "
          "When you have the answer, give it inside <answer> and </answer> without detailed illustrations.")


def to_row(ex, idx, split):
    answers = list(ex.get("golden_answers") or ex.get("answer") or [])
    src = f"searchR1_{ex.get('data_source', 'nq')}"
    return row(src, [{"role": "system", "content": SYSTEM}, {"role": "user", "content": ex["question"].strip()}], "fact-reasoning",
               {"target": answers}, split, idx, need_tools_kwargs=True,
               tools_kwargs={"search": {"create_kwargs": {"ground_truth": answers, "question": ex["question"], "data_source": src}}})


if __name__ == "__main__":
    build(parser("~/data/searchR1_processed_direct", __doc__).parse_args(), DATA_SOURCE, to_row)
