"""Write the fully composed trainer configurations next to their sources.

``python -m verl_b200.scripts.generate_trainer_config [--check]`` composes ``ppo_trainer.yaml`` for each engine family
(``model_engine=dp`` → ``_generated_ppo_trainer.yaml``, ``model_engine=megatron`` → ``_generated_ppo_megatron_trainer.yaml``)
WITHOUT resolving interpolations, so that the files show every key, its default and where it takes its value from. With
``--check`` nothing is written and the exit code says whether the committed files are current (used by the tests).
Reference: ``scripts/generate_trainer_config.sh`` and the ``_generated_*.yaml`` files of ``verl/trainer/config``.
"""

from __future__ import annotations

import argparse
import os
import sys

import yaml

from verl_b200.utils.config import _load_yaml_with_defaults

CONFIG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "trainer", "config")
TARGETS = {"_generated_ppo_trainer.yaml": {"model_engine": "dp"}, "_generated_ppo_megatron_trainer.yaml": {"model_engine": "megatron"}}
HEADER = ("# This file is generated: it is ppo_trainer.yaml with its `defaults` list composed ({choice}).\n"
          "# Do not edit it; change the group files and run `python -m verl_b200.scripts.generate_trainer_config`.\n")


def render(choices: dict) -> str:
    data = _load_yaml_with_defaults(os.path.join(CONFIG_DIR, "ppo_trainer.yaml"), dict(choices))
    body = yaml.safe_dump(data, sort_keys=False, default_flow_style=False, width=120)
    return HEADER.format(choice=", ".join(f"{k}={v}" for k, v in choices.items())) + body


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--check", action="store_true", help="only report whether the generated files are current")
    args = ap.parse_args(argv)
    stale = []
    for name, choices in TARGETS.items():
        path, text = os.path.join(CONFIG_DIR, name), render(choices)
        if args.check:
            if not os.path.exists(path) or open(path).read() != text:
                stale.append(name)
        else:
            with open(path, "w") as f:
                f.write(text)
            print(f"wrote {path}")
    if stale:
        print(f"stale generated configs: {stale}; run python -m verl_b200.scripts.generate_trainer_config", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
