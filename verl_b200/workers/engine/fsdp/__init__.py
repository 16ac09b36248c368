from .engine import FlatParamStore, FSDPEngine, FSDPEngineWithValueHead  # noqa: F401
