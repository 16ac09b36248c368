from .naive_rollout import HFRollout, NaiveRollout

__all__ = ["NaiveRollout", "HFRollout"]
