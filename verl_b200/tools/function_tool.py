"""Turn a plain Python function into a tool: the schema comes from its signature, type hints and docstring
(reference: ``verl/tools/function_tool.py:45``)."""

from __future__ import annotations

import asyncio
import inspect
import json
from typing import Any, Callable, Optional, get_type_hints

from .base_tool import BaseTool
from .schemas import OpenAIFunctionParametersSchema, OpenAIFunctionSchema, OpenAIFunctionToolSchema, ToolResponse

__all__ = ["FunctionTool", "function_to_schema"]

_JSON_TYPES = {int: "integer", float: "number", str: "string", bool: "boolean", list: "array", dict: "object"}


def _param_docs(doc: str) -> dict:
    """``name: text`` / ``name (type): text`` lines of a Google-style ``Args:`` block."""
    out, in_args = {}, False
    for line in (doc or "").splitlines():
        s = line.strip()
        if s.lower() in ("args:", "arguments:", "parameters:"):
            in_args = True
            continue
        if in_args:
            if not s or s.lower() in ("returns:", "raises:", "yields:"):
                in_args = False
                continue
            if ":" in s:
                k, v = s.split(":", 1)
                out[k.split("(")[0].strip()] = v.strip()
    return out


def function_to_schema(fn: Callable, name: Optional[str] = None, description: Optional[str] = None) -> OpenAIFunctionToolSchema:
    sig = inspect.signature(fn)
    hints = get_type_hints(fn)
    doc = inspect.getdoc(fn) or ""
    pdocs = _param_docs(doc)
    props, required = {}, []
    for pname, p in sig.parameters.items():
        if pname in ("self", "cls") or p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            continue
        t = hints.get(pname, str)
        origin = getattr(t, "__origin__", None)
        entry = {"type": _JSON_TYPES.get(origin or t, "string")}
        if pname in pdocs:
            entry["description"] = pdocs[pname]
        props[pname] = entry
        if p.default is inspect.Parameter.empty:
            required.append(pname)
    summary = description or doc.split("\n\n")[0].strip()
    return OpenAIFunctionToolSchema(function=OpenAIFunctionSchema(name=name or fn.__name__, description=summary,
                                                                  parameters=OpenAIFunctionParametersSchema(properties=props, required=required)))


class FunctionTool(BaseTool):
    def __init__(self, fn: Callable, name: Optional[str] = None, description: Optional[str] = None, config: Optional[dict] = None):
        self.fn = fn
        super().__init__(config, function_to_schema(fn, name, description))

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs) -> tuple[ToolResponse, float, dict]:
        try:
            res = self.fn(**parameters)
            if asyncio.iscoroutine(res):
                res = await res
        except Exception as e:  # noqa: BLE001 - the error text is what the model sees
            return ToolResponse(text=f"Error when executing tool: {type(e).__name__}: {e}"), 0.0, {"tool_error": 1}
        text = res if isinstance(res, str) else json.dumps(res, ensure_ascii=False, default=str)
        return ToolResponse(text=text), 0.0, {}
