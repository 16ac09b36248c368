"""Browse the trajectories a training run dumped with ``trainer.rollout_data_dir`` / ``trainer.validation_data_dir``.

    python -m verl_b200.scripts.rollout_viewer <dir> [--step N] [--sort=score|-score|length|-length] [--grep REGEX]
                                                [--min-score X] [--max-score X] [--limit K] [--field output] [--stats]

Without ``--step`` the latest ``{step}.jsonl`` is shown. ``--stats`` prints per-step counts, mean score and mean output
length for every dumped step instead of trajectories. Plain text on stdout (pipe it into a pager).

Reference: ``scripts/rollout_viewer.py`` (a terminal UI over the same JSONL files).
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys

__all__ = ["load_step", "list_steps", "main"]


def list_steps(path: str) -> list[int]:
    return sorted(int(f[:-6]) for f in os.listdir(path) if f.endswith(".jsonl") and f[:-6].isdigit())


def load_step(path: str, step: int) -> list[dict]:
    with open(os.path.join(path, f"{step}.jsonl")) as f:
        return [json.loads(line) for line in f if line.strip()]


def _length(r: dict) -> int:
    o = r.get("output", "")
    return len(o)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("path")
    ap.add_argument("--step", type=int, default=None)
    ap.add_argument("--sort", default=None, choices=["score", "-score", "length", "-length"])
    ap.add_argument("--grep", default=None, help="keep trajectories whose input or output matches this regular expression")
    ap.add_argument("--min-score", type=float, default=None)
    ap.add_argument("--max-score", type=float, default=None)
    ap.add_argument("--limit", type=int, default=20)
    ap.add_argument("--field", action="append", default=None, help="fields to print (default: input, output, score and extras)")
    ap.add_argument("--stats", action="store_true")
    a = ap.parse_args(argv)
    steps = list_steps(a.path)
    if not steps:
        print(f"no {{step}}.jsonl files in {a.path}", file=sys.stderr)
        return 1
    if a.stats:
        print(f"{'step':>8} {'n':>6} {'mean score':>11} {'mean length':>12}")
        for s in steps:
            rows = load_step(a.path, s)
            n = max(1, len(rows))
            print(f"{s:>8} {len(rows):>6} {sum(r.get('score', 0.0) for r in rows) / n:>11.4f} {sum(_length(r) for r in rows) / n:>12.1f}")
        return 0
    step = a.step if a.step is not None else steps[-1]
    rows = load_step(a.path, step)
    if a.grep:
        rx = re.compile(a.grep)
        rows = [r for r in rows if rx.search(str(r.get("input", ""))) or rx.search(str(r.get("output", "")))]
    if a.min_score is not None:
        rows = [r for r in rows if r.get("score", 0.0) >= a.min_score]
    if a.max_score is not None:
        rows = [r for r in rows if r.get("score", 0.0) <= a.max_score]
    if a.sort:
        key = (lambda r: r.get("score", 0.0)) if "score" in a.sort else _length
        rows.sort(key=key, reverse=a.sort.startswith("-"))
    print(f"step {step}: {len(rows)} trajectories (showing {min(len(rows), a.limit)})")
    for i, r in enumerate(rows[: a.limit]):
        print("=" * 100)
        print(f"#{i}  score={r.get('score')}  source={r.get('data_source')}  gts={r.get('gts')}")
        fields = a.field or ["input", "output"] + [k for k in r if k not in ("input", "output", "score", "data_source", "gts", "step")]
        for k in fields:
            print(f"--- {k}")
            print(r.get(k))
    return 0


if __name__ == "__main__":
    sys.exit(main())
