"""Load tools from a yaml/dict description (reference: ``verl/tools/tool_registry.py:36`` ``initialize_tools_from_config``).

    tools:
      - class_name: "my_pkg.tools.SearchTool"          # BaseTool subclass, or
        config: {type: native, ...}
        tool_schema: {type: function, function: {...}}
      - function: "my_pkg.tools.calculator"            # plain function → FunctionTool
"""

from __future__ import annotations

from typing import Union

from verl_b200.utils.import_utils import load_class_from_fqn

from .base_tool import BaseTool
from .function_tool import FunctionTool
from .schemas import OpenAIFunctionToolSchema

__all__ = ["initialize_tools_from_config", "get_tool_class", "register_tool", "TOOL_REGISTRY"]

TOOL_REGISTRY: dict[str, type] = {}


def register_tool(name: str):
    def deco(cls):
        TOOL_REGISTRY[name] = cls
        return cls

    return deco


def get_tool_class(name: str):
    if name in TOOL_REGISTRY:
        return TOOL_REGISTRY[name]
    return load_class_from_fqn(name)


def initialize_tools_from_config(config: Union[str, dict, list]) -> list[BaseTool]:
    if isinstance(config, str):
        import yaml

        with open(config) as f:
            config = yaml.safe_load(f)
    entries = config.get("tools", []) if isinstance(config, dict) else list(config)
    tools: list[BaseTool] = []
    for e in entries:
        if "function" in e and "class_name" not in e:
            fn = load_class_from_fqn(e["function"]) if isinstance(e["function"], str) else e["function"]
            tools.append(FunctionTool(fn, name=e.get("name"), description=e.get("description"), config=e.get("config")))
            continue
        cls = get_tool_class(e["class_name"])
        schema = OpenAIFunctionToolSchema.from_dict(e["tool_schema"]) if e.get("tool_schema") else None
        tools.append(cls(config=e.get("config", {}), tool_schema=schema))
    return tools
