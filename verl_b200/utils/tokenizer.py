"""Tokenizer helpers: HF loading with the pad-token fix-up of the reference (``verl/utils/tokenizer.py``) and a
dependency-free byte-level chat tokenizer for offline runs, synthetic benchmarks and tests.
"""

from __future__ import annotations

import json
from typing import Optional

__all__ = ["hf_tokenizer", "ByteChatTokenizer"]


def hf_tokenizer(path: str, correct_pad_token: bool = True, **kwargs):
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(path, **kwargs)
    if correct_pad_token and tok.pad_token_id is None:
        tok.pad_token_id = tok.eos_token_id
        tok.pad_token = tok.eos_token
    return tok


class ByteChatTokenizer:
    """UTF-8 bytes (ids 0..255) plus a few specials; ChatML-like template

        <|im_start|>role\\ncontent<|im_end|>\\n ... <|im_start|>assistant\\n

    Tools are listed in the system turn as JSON lines; tool results use the ``tool`` role. Implements the subset of the
    HF tokenizer interface the framework uses: ``__call__``, ``encode``, ``decode``, ``apply_chat_template``.
    """

    SPECIALS = ["<|pad|>", "<|im_start|>", "<|im_end|>", "<|endoftext|>"]

    def __init__(self, vocab_size: int = 260):
        assert vocab_size >= 256 + len(self.SPECIALS)
        self.vocab_size = vocab_size
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.pad_token_id, self.eos_token_id = self.special_ids["<|pad|>"], self.special_ids["<|im_end|>"]
        self.pad_token, self.eos_token = "<|pad|>", "<|im_end|>"
        self.padding_side = "left"

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        out, i = [], 0
        while i < len(text):
            for s, sid in self.special_ids.items():
                if text.startswith(s, i):
                    out.append(sid)
                    i += len(s)
                    break
            else:
                j = i + 1
                while j < len(text) and not any(text.startswith(s, j) for s in self.special_ids):
                    j += 1
                out.extend(text[i:j].encode("utf-8"))
                i = j
        return out

    def __call__(self, text, add_special_tokens: bool = False, **kwargs):
        if isinstance(text, str):
            return {"input_ids": self.encode(text), "attention_mask": [1] * len(self.encode(text))}
        ids = [self.encode(t) for t in text]
        return {"input_ids": ids, "attention_mask": [[1] * len(x) for x in ids]}

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        inv = {v: k for k, v in self.special_ids.items()}
        parts, buf = [], bytearray()
        for t in ids:
            t = int(t)
            if t < 256:
                buf.append(t)
            else:
                if buf:
                    parts.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                if not skip_special_tokens and t in inv:
                    parts.append(inv[t])
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)

    def batch_decode(self, seqs, skip_special_tokens: bool = False):
        return [self.decode(s, skip_special_tokens) for s in seqs]

    def apply_chat_template(self, messages, tools: Optional[list] = None, add_generation_prompt: bool = True, tokenize: bool = True, **kwargs):
        text = ""
        msgs = list(messages)
        if tools:
            desc = "# Tools\n" + "\n".join(json.dumps(t, ensure_ascii=False) for t in tools) + \
                   '\nCall a tool with <tool_call>{"name": ..., "arguments": {...}}</tool_call>'
            if msgs and msgs[0]["role"] == "system":
                msgs[0] = {"role": "system", "content": msgs[0]["content"] + "\n\n" + desc}
            else:
                msgs.insert(0, {"role": "system", "content": desc})
        for m in msgs:
            content = m.get("content") or ""
            if not isinstance(content, str):
                content = "".join(c.get("text", "") for c in content if isinstance(c, dict))
            text += f"<|im_start|>{m['role']}\n{content}<|im_end|>\n"
        if add_generation_prompt:
            text += "<|im_start|>assistant\n"
        return self.encode(text) if tokenize else text
