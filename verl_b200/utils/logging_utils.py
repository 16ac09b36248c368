"""Process-wide logging setup (reference: ``verl/utils/logging_utils.py:22-46``).

``VERL_LOGGING_LEVEL`` (default INFO) sets the level of the package logger, which gets its own stderr handler and does not propagate, so a
library that reconfigures the root logger (an inference server, a tokenizer) neither silences nor duplicates the framework's lines.
"""
from __future__ import annotations

import logging
import os
import sys

import torch.distributed as dist

_FORMAT = "%(levelname)s:%(asctime)s:%(message)s"
PACKAGE_LOGGER = "verl_b200"


def configure_verl_logging(name: str = PACKAGE_LOGGER) -> logging.Logger:
    level = os.getenv("VERL_LOGGING_LEVEL", "INFO").upper()
    handler = logging.StreamHandler(stream=sys.stderr)
    handler.setLevel(level)
    handler.setFormatter(logging.Formatter(_FORMAT))
    lg = logging.getLogger(name)
    lg.handlers = [handler]
    lg.setLevel(level)
    lg.propagate = False
    return lg


def set_basic_config(level) -> None:
    logging.basicConfig(format=_FORMAT, level=level)


def log_to_file(string: str, directory: str = "logs") -> None:
    """Prints, and appends to ``<directory>/log_<rank>`` when that directory exists."""
    print(string)
    if os.path.isdir(directory):
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        with open(os.path.join(directory, f"log_{rank}"), "a+") as f:
            f.write(string + "\n")
