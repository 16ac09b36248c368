"""Extract function calls from generated text. One parser per chat-template family, registered by name
(reference: ``verl/experimental/agent_loop/tool_parser.py:48-743``).

``extract_tool_calls(text)`` returns ``(content_without_calls, [FunctionCall])``; malformed calls are skipped.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass

__all__ = ["FunctionCall", "ToolParser", "HermesToolParser", "Qwen3XMLToolParser", "GptOssToolParser", "get_tool_parser"]


@dataclass
class FunctionCall:
    name: str
    arguments: str     # JSON text, as in the OpenAI API


class ToolParser:
    _registry: dict[str, type] = {}

    @classmethod
    def register(cls, name: str):
        def deco(sub):
            cls._registry[name] = sub
            return sub

        return deco

    @classmethod
    def get_tool_parser(cls, name: str, tokenizer=None) -> "ToolParser":
        if name not in cls._registry:
            raise ValueError(f"unknown tool parser {name!r}; known: {sorted(cls._registry)}")
        return cls._registry[name](tokenizer)

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer

    def extract_tool_calls(self, text: str) -> tuple[str, list[FunctionCall]]:
        raise NotImplementedError

    async def extract_tool_calls_from_ids(self, token_ids: list) -> tuple[str, list[FunctionCall]]:
        return self.extract_tool_calls(self.tokenizer.decode(token_ids))


@ToolParser.register("hermes")
class HermesToolParser(ToolParser):
    """``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (Qwen2.5 / Hermes templates)."""

    _re = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)

    def extract_tool_calls(self, text: str):
        calls = []
        for m in self._re.findall(text):
            try:
                d = json.loads(m)
                calls.append(FunctionCall(name=d["name"], arguments=json.dumps(d.get("arguments", {}), ensure_ascii=False)))
            except (json.JSONDecodeError, KeyError, TypeError):
                continue
        return self._re.sub("", text), calls


@ToolParser.register("qwen3_xml")
class Qwen3XMLToolParser(ToolParser):
    """``<tool_call><function=name><parameter=key>value</parameter>…</function></tool_call>`` (Qwen3-Coder style)."""

    _call = re.compile(r"<tool_call>\s*<function=([^>]+)>(.*?)</function>\s*</tool_call>", re.DOTALL)
    _param = re.compile(r"<parameter=([^>]+)>(.*?)</parameter>", re.DOTALL)

    def extract_tool_calls(self, text: str):
        calls = []
        for name, body in self._call.findall(text):
            args = {}
            for k, v in self._param.findall(body):
                v = v.strip()
                try:
                    args[k.strip()] = json.loads(v)
                except json.JSONDecodeError:
                    args[k.strip()] = v
            calls.append(FunctionCall(name=name.strip(), arguments=json.dumps(args, ensure_ascii=False)))
        return self._call.sub("", text), calls


@ToolParser.register("gpt-oss")
class GptOssToolParser(ToolParser):
    """Harmony format: ``<|start|>assistant<|channel|>commentary to=functions.NAME <|constrain|>json<|message|>{...}<|call|>``."""

    _re = re.compile(r"to=functions\.([\w\-.]+)[^<]*(?:<\|constrain\|>\w+)?<\|message\|>(.*?)<\|call\|>", re.DOTALL)

    def extract_tool_calls(self, text: str):
        calls = []
        for name, body in self._re.findall(text):
            try:
                calls.append(FunctionCall(name=name, arguments=json.dumps(json.loads(body), ensure_ascii=False)))
            except json.JSONDecodeError:
                continue
        return self._re.sub("", text), calls


def get_tool_parser(name: str, tokenizer=None) -> ToolParser:
    return ToolParser.get_tool_parser(name, tokenizer)
