"""Print the fully resolved trainer config: ``python -m verl_b200.scripts.print_cfg [ppo_trainer] key=value ...``
(reference: ``scripts/print_cfg.py``)."""

import sys

import yaml

from verl_b200.utils.config import load_config
from verl_b200.utils.py_functional import convert_to_regular_types


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    name = argv.pop(0) if argv and "=" not in argv[0] else "ppo_trainer"
    cfg = load_config(name, argv)
    print(yaml.safe_dump(convert_to_regular_types(cfg), sort_keys=False))


if __name__ == "__main__":
    main()
