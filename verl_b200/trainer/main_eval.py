"""Offline evaluation of a generations file: ``python -m verl_b200.trainer.main_eval data.path=gen.parquet
[data.prompt_key=prompt data.response_key=responses data.data_source_key=data_source data.reward_model_key=reward_model]
[custom_reward_function.path=f.py custom_reward_function.name=compute_score]``

Every row holds one prompt with a list of sampled responses; each response is scored with the rule for the row's data
source (or the custom function) in a process pool and the mean of the per-prompt means is reported per data source as
``test_score/<source>`` (reference: ``verl/trainer/main_eval.py:34-80`` does the same with Ray tasks).
"""

from __future__ import annotations

import concurrent.futures
import sys
from collections import defaultdict

import numpy as np

from verl_b200.utils.config import Config, apply_overrides

DEFAULT = {"data": {"path": None, "prompt_key": "prompt", "response_key": "responses", "data_source_key": "data_source",
                    "reward_model_key": "reward_model"}, "custom_reward_function": {"path": None, "name": "compute_score"}, "num_workers": 8}


def _score_row(args):
    data_source, responses, ground_truth, fn_path, fn_name = args
    if fn_path:
        from verl_b200.utils.import_utils import load_extern_type

        fn = load_extern_type(fn_path, fn_name)
    else:
        from verl_b200.utils.reward_score import default_compute_score as fn
    scores = []
    for r in responses:
        s = fn(data_source, r, ground_truth) if not fn_path else fn(data_source=data_source, solution_str=r, ground_truth=ground_truth)
        scores.append(float(s["score"] if isinstance(s, dict) else s))
    return data_source, float(np.mean(scores)) if scores else 0.0


def evaluate(cfg: Config) -> dict:
    import pandas as pd

    df = pd.read_parquet(cfg.data.path)
    rows = []
    for _, r in df.iterrows():
        rm = r[cfg.data.reward_model_key]
        gt = rm["ground_truth"] if hasattr(rm, "__getitem__") and "ground_truth" in rm else rm
        rows.append((r[cfg.data.data_source_key], list(r[cfg.data.response_key]), gt, cfg.custom_reward_function.path, cfg.custom_reward_function.name))
    by_source = defaultdict(list)
    workers = int(cfg.get("num_workers", 8))
    if workers > 1 and len(rows) > 16:
        with concurrent.futures.ProcessPoolExecutor(workers) as ex:
            results = list(ex.map(_score_row, rows, chunksize=16))
    else:
        results = [_score_row(r) for r in rows]
    for src, s in results:
        by_source[src].append(s)
    return {f"test_score/{k}": float(np.mean(v)) for k, v in by_source.items()}


def main(argv=None):
    import copy

    data = copy.deepcopy(DEFAULT)
    apply_overrides(data, list(sys.argv[1:] if argv is None else argv))
    metrics = evaluate(Config(data))
    print(metrics)
    return metrics


if __name__ == "__main__":
    main()
