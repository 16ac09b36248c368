"""OpenAI function-calling schemas as plain dataclasses (reference: ``verl/tools/schemas.py`` pydantic models)."""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Optional

__all__ = ["OpenAIFunctionParametersSchema", "OpenAIFunctionSchema", "OpenAIFunctionToolSchema", "OpenAIFunctionCallSchema",
           "OpenAIFunctionToolCall", "ToolResponse"]


@dataclass
class OpenAIFunctionParametersSchema:
    type: str = "object"
    properties: dict = field(default_factory=dict)
    required: list = field(default_factory=list)


@dataclass
class OpenAIFunctionSchema:
    name: str
    description: str = ""
    parameters: OpenAIFunctionParametersSchema = field(default_factory=OpenAIFunctionParametersSchema)
    strict: bool = False


@dataclass
class OpenAIFunctionToolSchema:
    type: str = "function"
    function: Optional[OpenAIFunctionSchema] = None

    @classmethod
    def from_dict(cls, d: dict) -> "OpenAIFunctionToolSchema":
        fn = d["function"]
        params = fn.get("parameters", {}) or {}
        return cls(type=d.get("type", "function"),
                   function=OpenAIFunctionSchema(name=fn["name"], description=fn.get("description", ""), strict=fn.get("strict", False),
                                                 parameters=OpenAIFunctionParametersSchema(type=params.get("type", "object"),
                                                                                           properties=params.get("properties", {}),
                                                                                           required=params.get("required", []))))

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass
class OpenAIFunctionCallSchema:
    name: str
    arguments: dict

    @staticmethod
    def from_openai_function_parsed_schema(name: str, arguments: Any) -> tuple["OpenAIFunctionCallSchema", bool]:
        """Returns (schema, has_decode_error): arguments may arrive as a JSON string."""
        import json

        err = False
        if isinstance(arguments, str):
            try:
                arguments = json.loads(arguments)
            except json.JSONDecodeError:
                arguments, err = {}, True
        if not isinstance(arguments, dict):
            arguments, err = {}, True
        return OpenAIFunctionCallSchema(name=name, arguments=arguments), err


@dataclass
class OpenAIFunctionToolCall:
    id: str
    function: OpenAIFunctionCallSchema
    type: str = "function"


@dataclass
class ToolResponse:
    text: Optional[str] = None
    image: Optional[list] = None
    video: Optional[list] = None

    def is_text_only(self) -> bool:
        return not self.image and not self.video
