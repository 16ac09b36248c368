from .registry import REWARD_MANAGER_REGISTRY, get_reward_manager_cls, register  # noqa: F401
from . import naive, batch, dapo, prime, token_rule  # noqa: F401,E402
