from .base_tool import BaseTool
from .function_tool import FunctionTool, function_to_schema
from .schemas import (OpenAIFunctionCallSchema, OpenAIFunctionParametersSchema, OpenAIFunctionSchema, OpenAIFunctionToolCall,
                      OpenAIFunctionToolSchema, ToolResponse)
from .tool_registry import initialize_tools_from_config, register_tool

__all__ = ["BaseTool", "FunctionTool", "function_to_schema", "OpenAIFunctionCallSchema", "OpenAIFunctionParametersSchema",
           "OpenAIFunctionSchema", "OpenAIFunctionToolCall", "OpenAIFunctionToolSchema", "ToolResponse",
           "initialize_tools_from_config", "register_tool"]
