"""Check that a tokenizer's chat template can be continued token by token (what multi-turn rollouts rely on).

    python -m verl_b200.scripts.chat_template_checker --model <dir with tokenizer files> [--template chat_template.jinja]

Prints one line per mock conversation and exits 1 if the token-level builder check fails for any of them (a failing raw
prefix diagnostic alone is reported as a warning). Without ``--model`` the built-in byte-level chat tokenizer is checked.

Reference: ``scripts/chat_template_checker.py`` + ``scripts/chat_template_mock_trajectories.py``.
"""

from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default=None, help="directory with tokenizer files (local only)")
    ap.add_argument("--template", default=None, help="file with a chat template to use instead of the tokenizer's own")
    ap.add_argument("--trajectories", default=None, help="JSON file {name: [messages...]} replacing the built-in conversations")
    a = ap.parse_args(argv)
    from verl_b200.utils.continuous_token import MOCK_TRAJECTORIES, check_append_only

    if a.model:
        from verl_b200.utils.tokenizer import hf_tokenizer

        tok = hf_tokenizer(a.model)
    else:
        from verl_b200.utils.tokenizer import ByteChatTokenizer

        tok = ByteChatTokenizer()
    if a.template:
        with open(a.template) as f:
            tok.chat_template = f.read()
    traj = MOCK_TRAJECTORIES
    if a.trajectories:
        with open(a.trajectories) as f:
            traj = json.load(f)
    report = check_append_only(tok, traj)
    bad = 0
    for name, r in report.items():
        status = "ok" if r["builder"] else "FAIL"
        warn = "" if r["raw_prefix"] else "  (warning: raw template is not append-only)"
        print(f"{name:24s} builder={status} boundaries={r['boundaries']}{warn}{'  ' + r['detail'] if r['detail'] else ''}")
        bad += not r["builder"]
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
