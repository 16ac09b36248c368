from .engine import MegatronEngine, MegatronEngineWithValueHead  # noqa: F401
