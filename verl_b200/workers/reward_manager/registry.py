"""String → reward-manager class (reference: ``verl/workers/reward_manager/registry.py``)."""

REWARD_MANAGER_REGISTRY: dict = {}


def register(name: str):
    def deco(cls):
        if name in REWARD_MANAGER_REGISTRY and REWARD_MANAGER_REGISTRY[name] is not cls:
            raise ValueError(f"reward manager {name} already registered")
        REWARD_MANAGER_REGISTRY[name] = cls
        return cls

    return deco


def get_reward_manager_cls(name: str):
    if name not in REWARD_MANAGER_REGISTRY:
        raise ValueError(f"Unknown reward manager: {name}; known: {sorted(REWARD_MANAGER_REGISTRY)}")
    return REWARD_MANAGER_REGISTRY[name]
