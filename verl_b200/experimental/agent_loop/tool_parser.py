"""Extract function calls from generated text. One parser per chat-template family, registered by name
(reference: ``verl/experimental/agent_loop/tool_parser.py:48-743``).

``extract_tool_calls(text)`` returns ``(content_without_calls, [FunctionCall])``; malformed calls are skipped.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass

__all__ = ["FunctionCall", "ToolParser", "HermesToolParser", "Qwen3XMLToolParser", "GptOssToolParser", "GLMToolParser", "SeedToolParser",
           "MiniMaxToolParser", "KimiToolParser", "DeepSeekV4ToolParser", "Gemma4ToolParser", "get_tool_parser"]


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

    @property
    def stop_token_ids(self) -> list[int]:
        """Extra token ids that end a tool-calling turn for this template family (besides EOS)."""
        tok = getattr(self, "stop_token", None)
        if tok is None or self.tokenizer is None or not hasattr(self.tokenizer, "convert_tokens_to_ids"):
            return []
        tid = self.tokenizer.convert_tokens_to_ids(tok)
        return [tid] if isinstance(tid, int) and tid >= 0 else []


def _json_or_text(raw: str):
    v = raw.strip()
    try:
        return json.loads(v)
    except (json.JSONDecodeError, ValueError):
        return v


def _dumps(args: dict) -> str:
    return json.dumps(args, ensure_ascii=False)


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


ToolParser._registry["qwen3_coder"] = Qwen3XMLToolParser      # the reference's name for the same format


class _BlockToolParser(ToolParser):
    """Calls wrapped in an outer block; ``_call`` finds (name, body) pairs inside a block, ``_arg`` (key, value) pairs in a body."""

    _block: re.Pattern
    _call: re.Pattern
    _arg: re.Pattern

    def extract_tool_calls(self, text: str):
        calls = []
        for block in self._block.findall(text):
            for name, body in self._call.findall(block):
                calls.append(FunctionCall(name=name.strip(), arguments=_dumps({k.strip(): _json_or_text(v) for k, v in self._arg.findall(body)})))
        return self._block.sub("", text), calls


@ToolParser.register("seed")
class SeedToolParser(_BlockToolParser):
    """``<seed:tool_call><function=NAME><parameter=KEY>VALUE</parameter>…</function></seed:tool_call>`` (ByteDance Seed)."""

    _block = re.compile(r"<seed:tool_call>(.*?)</seed:tool_call>", re.DOTALL)
    _call = re.compile(r"<function=([^>\n]+)>\s*(.*?)</function>", re.DOTALL)
    _arg = re.compile(r"<parameter=([^>\n]+)>(.*?)</parameter>", re.DOTALL)


@ToolParser.register("minimax")
class MiniMaxToolParser(_BlockToolParser):
    """``<minimax:tool_call><invoke name="NAME"><parameter name="KEY">VALUE</parameter>…</invoke></minimax:tool_call>``."""

    _block = re.compile(r"<minimax:tool_call>(.*?)</minimax:tool_call>", re.DOTALL)
    _call = re.compile(r'<invoke name="([^"]+)">\s*(.*?)</invoke>', re.DOTALL)
    _arg = re.compile(r'<parameter name="([^"]+)">(.*?)</parameter>', re.DOTALL)


@ToolParser.register("glm")
class GLMToolParser(ToolParser):
    """``<tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value>…</tool_call>``; the turn ends at ``<|observation|>``."""

    stop_token = "<|observation|>"
    _re = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)
    _pair = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.DOTALL)

    def extract_tool_calls(self, text: str):
        calls = []
        for body in self._re.findall(text):
            i = body.find("<arg_key>")
            name = (body if i < 0 else body[:i]).strip()
            if not name:
                continue
            args = {} if i < 0 else {k.strip(): _json_or_text(v) for k, v in self._pair.findall(body[i:])}
            calls.append(FunctionCall(name=name, arguments=_dumps(args)))
        return self._re.sub("", text), calls


@ToolParser.register("kimi")
class KimiToolParser(ToolParser):
    """Kimi K2 special tokens: ``<|tool_calls_section_begin|><|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{json}
    <|tool_call_end|>…<|tool_calls_section_end|>``; the id prefix ``functions.`` and the ``:IDX`` suffix are stripped."""

    stop_token = "<|im_end|>"
    _section = re.compile(r"<\|tool_calls_section_begin\|>(.*?)(?:<\|tool_calls_section_end\|>|$)", re.DOTALL)
    _call = re.compile(r"<\|tool_call_begin\|>(.*?)<\|tool_call_argument_begin\|>(.*?)<\|tool_call_end\|>", re.DOTALL)

    def extract_tool_calls(self, text: str):
        calls = []
        for raw_name, raw_args in self._call.findall(text):
            name = raw_name.strip()
            if name.startswith("functions."):
                name = name[len("functions."):]
            name = re.sub(r":\d+$", "", name)
            args = _json_or_text(raw_args)
            calls.append(FunctionCall(name=name, arguments=_dumps(args if isinstance(args, dict) else {})))
        return self._section.sub("", text), calls


@ToolParser.register("deepseek_v4")
class DeepSeekV4ToolParser(ToolParser):
    """DSML blocks: ``<｜DSML｜tool_calls><｜DSML｜invoke name="NAME"><｜DSML｜parameter name="K" string="true|false">V</｜DSML｜parameter>
    …</｜DSML｜invoke></｜DSML｜tool_calls>``; ``string="true"`` keeps the raw text, ``"false"`` parses JSON."""

    _d = re.escape("｜DSML｜")
    _block = re.compile(rf"<{_d}tool_calls>(.*?)</{_d}tool_calls>", re.DOTALL)
    _call = re.compile(rf'<{_d}invoke name="(.*?)">(.*?)</{_d}invoke>', re.DOTALL)
    _arg = re.compile(rf'<{_d}parameter name="(.*?)" string="(true|false)">(.*?)</{_d}parameter>', re.DOTALL)

    def extract_tool_calls(self, text: str):
        calls = []
        for block in self._block.findall(text):
            for name, body in self._call.findall(block):
                args = {k: (v if is_str == "true" else _json_or_text(v)) for k, is_str, v in self._arg.findall(body)}
                calls.append(FunctionCall(name=name.strip(), arguments=_dumps(args)))
        return self._block.sub("", text), calls


@ToolParser.register("gemma4")
class Gemma4ToolParser(ToolParser):
    """``<|tool_call>call:NAME{key:<|"|>text<|"|>,n:3,flag:true}<tool_call|>``; generation stops at ``<tool_call|>`` so the tool
    can run between calls."""

    stop_token = "<tool_call|>"
    _re = re.compile(r"<\|tool_call>call:(\w+)\{(.*?)\}<tool_call\|>", re.DOTALL)
    _arg = re.compile(r'(\w+):(?:<\|"\|>(.*?)<\|"\|>|([^,}]*))', re.DOTALL)

    @staticmethod
    def _bare(v: str):
        v = v.strip()
        low = v.lower()
        if low in ("true", "false"):
            return low == "true"
        if low == "null":
            return None
        for cast in (int, float):
            try:
                return cast(v)
            except ValueError:
                pass
        return v

    def extract_tool_calls(self, text: str):
        calls = []
        for name, body in self._re.findall(text):
            args = {}
            for m in self._arg.finditer(body):
                args[m.group(1)] = m.group(2) if m.group(2) is not None else self._bare(m.group(3) or "")
            calls.append(FunctionCall(name=name, arguments=_dumps(args)))
        return self._re.sub("", text), calls


def get_tool_parser(name: str, tokenizer=None) -> ToolParser:
    return ToolParser.get_tool_parser(name, tokenizer)
