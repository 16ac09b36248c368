"""Shared pieces of the dataset preparation scripts: read a raw dataset (a local directory of ``{split}.jsonl|json|parquet`` files,
or a Hugging Face dataset name when the ``datasets`` package and a network are available), map every example to the training
schema, write ``train.parquet`` / ``test.parquet``.

Training schema (one row per prompt; what ``verl_b200.utils.dataset.RLHFDataset`` reads):
``data_source`` (selects the scorer), ``prompt`` (chat messages), ``ability``, ``reward_model`` = ``{"style", "ground_truth"}``,
``extra_info`` (``split``, ``index``, optional ``tools_kwargs`` / ``interaction_kwargs`` for multi-turn rollouts), optional ``images``.

Reference: ``examples/data_preprocess/*.py`` of the reference (one stand-alone script per dataset built on ``datasets.map``); here
one loader / writer is shared and each script only holds its example → row function.
"""

from __future__ import annotations

import argparse
import json
import os
from typing import Callable, Iterable, Optional

import pandas as pd


def parser(default_save_dir: str, description: str = "") -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--local_dataset_path", default=None, help="directory (or file stem) holding the raw {split}.jsonl / .json / .parquet files")
    ap.add_argument("--local_save_dir", default=default_save_dir, help="where train.parquet / test.parquet are written")
    ap.add_argument("--local_dir", default=None, help="deprecated alias of --local_save_dir")
    ap.add_argument("--hdfs_dir", default=None, help="copy the result there as well (verl_b200.utils.fs.copy)")
    ap.add_argument("--max_rows", type=int, default=0, help="keep only the first N examples of every split (0 = all)")
    return ap


def load_split(source: Optional[str], hub_name: str, split: str, hub_config: Optional[str] = None) -> list[dict]:
    """Examples of one split as plain dicts."""
    if source:
        src = os.path.expanduser(source)
        cands = [os.path.join(src, f"{split}{ext}") for ext in (".jsonl", ".json", ".parquet")] if os.path.isdir(src) else [src]
        for c in cands:
            if not os.path.exists(c):
                continue
            if c.endswith(".parquet"):
                return pd.read_parquet(c).to_dict("records")
            with open(c) as f:
                if c.endswith(".jsonl"):
                    return [json.loads(line) for line in f if line.strip()]
                data = json.load(f)
                return data if isinstance(data, list) else data[split]
        raise FileNotFoundError(f"no {split}.jsonl / .json / .parquet under {src}")
    try:
        import datasets
    except ImportError as e:  # noqa: F841
        raise SystemExit(f"the `datasets` package is not installed: pass --local_dataset_path with the raw {hub_name} files") from None
    ds = datasets.load_dataset(hub_name, hub_config) if hub_config else datasets.load_dataset(hub_name)
    return [dict(r) for r in ds[split]]


def build(args, hub_name: str, row_fn: Callable[[dict, int, str], Optional[dict]], splits: Iterable[str] = ("train", "test"),
          hub_config: Optional[str] = None, split_alias: Optional[dict] = None) -> dict:
    """Map every split through ``row_fn(example, index, split)`` (``None`` drops the example) and write the parquet files.
    Returns ``{split: path}``."""
    out_dir = os.path.expanduser(args.local_dir or args.local_save_dir)
    os.makedirs(out_dir, exist_ok=True)
    written = {}
    for split in splits:
        raw = load_split(args.local_dataset_path, hub_name, (split_alias or {}).get(split, split), hub_config)
        if args.max_rows:
            raw = raw[: args.max_rows]
        rows = [r for r in (row_fn(dict(ex), i, split) for i, ex in enumerate(raw)) if r is not None]
        path = os.path.join(out_dir, f"{split}.parquet")
        pd.DataFrame(rows).to_parquet(path)
        written[split] = path
        print(f"{split}: {len(rows)} rows -> {path}")
    if args.hdfs_dir:
        from verl_b200.utils.fs import copy

        copy(out_dir, args.hdfs_dir)
    return written


def row(data_source: str, messages: list, ability: str, ground_truth, split: str, index: int, style: str = "rule", **extra) -> dict:
    images = extra.pop("images", None)
    r = {"data_source": data_source, "prompt": messages, "ability": ability, "reward_model": {"style": style, "ground_truth": ground_truth},
         "extra_info": {"split": split, "index": index, **extra}}
    if images is not None:
        r["images"] = images
    return r
