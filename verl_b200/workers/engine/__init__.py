from .base import BaseEngine, BaseEngineCtx, EngineRegistry  # noqa: F401
