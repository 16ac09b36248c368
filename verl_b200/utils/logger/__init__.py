"""Rank-aware console logging helpers (reference: ``verl/utils/logger/__init__.py``, ``aggregate_logger.py:26-140``)."""
from verl_b200.utils.logger.aggregate_logger import (DecoratorLoggerBase, LocalLogger, concat_dict_to_str, log_with_rank, print_rank_0,
                                                     print_with_rank, print_with_rank_and_timer)

__all__ = ["LocalLogger", "DecoratorLoggerBase", "concat_dict_to_str", "print_rank_0", "print_with_rank", "print_with_rank_and_timer",
           "log_with_rank"]
