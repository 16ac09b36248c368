"""Tool contract of multi-turn rollouts (reference: ``verl/tools/base_tool.py:24-94``): per-trajectory instances with
``create`` → ``execute``* → ``calc_reward`` → ``release``."""

from __future__ import annotations

import uuid
from typing import Any, Optional

from .schemas import OpenAIFunctionToolSchema, ToolResponse

__all__ = ["BaseTool"]


class BaseTool:
    def __init__(self, config: Optional[dict] = None, tool_schema: Optional[OpenAIFunctionToolSchema] = None):
        self.config = config or {}
        self.tool_schema = tool_schema or self.get_openai_tool_schema()
        assert self.tool_schema is not None, "a tool needs a schema"
        self.name = self.tool_schema.function.name

    def get_openai_tool_schema(self) -> Optional[OpenAIFunctionToolSchema]:
        return getattr(self, "tool_schema", None)

    async def create(self, instance_id: Optional[str] = None, **kwargs) -> tuple[str, ToolResponse]:
        return instance_id or uuid.uuid4().hex, ToolResponse()

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs) -> tuple[ToolResponse, float, dict]:
        """Returns (response shown to the model, step reward, metrics)."""
        return ToolResponse(text="Updated the tool state."), 0.0, {}

    async def calc_reward(self, instance_id: str, **kwargs) -> float:
        return 0.0

    async def release(self, instance_id: str, **kwargs) -> None:
        return None
