"""Datasets for supervised stages (reference: ``verl/utils/dataset/multiturn_sft_dataset.py``, ``rm_dataset.py``).

``MultiTurnSFTDataset`` tokenises chat transcripts turn by turn and builds a loss mask that is 1 only on assistant tokens
(including each assistant turn's end-of-turn token); ``RMDataset`` yields (chosen, rejected) token pairs for reward-model
training. Both pad/truncate to ``max_length`` and return the keys the trainers expect.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
from torch.utils.data import Dataset

from verl_b200.utils.torch_functional import compute_position_id_with_mask

__all__ = ["MultiTurnSFTDataset", "RMDataset"]


def _read(files):
    import pandas as pd

    files = [files] if isinstance(files, str) else list(files)
    return pd.concat([pd.read_parquet(os.path.expanduser(f)) for f in files], ignore_index=True)


def _ids(tok, messages, **kw):
    out = tok.apply_chat_template(messages, tokenize=True, **kw)
    return list(out["input_ids"] if isinstance(out, dict) else out)


class MultiTurnSFTDataset(Dataset):
    def __init__(self, files=None, tokenizer=None, max_length: int = 1024, messages_key: str = "messages", tools_key: str = "tools",
                 truncation: str = "right", rows: Optional[list] = None):
        assert truncation in ("right", "left", "error")
        self.tok, self.max_length, self.truncation = tokenizer, max_length, truncation
        if rows is None:
            df = _read(files)
            rows = [{"messages": list(r[messages_key]), "tools": (list(r[tools_key]) if tools_key in df.columns and r[tools_key] is not None else None)}
                    for _, r in df.iterrows()]
        self.rows = rows

    def __len__(self):
        return len(self.rows)

    def _tokenize(self, messages, tools):
        """Incremental templating: tokens of turn i = template(messages[:i+1]) minus template(messages[:i])."""
        ids, mask, prev = [], [], []
        for i, m in enumerate(messages):
            gen_prompt = []
            if m["role"] == "assistant":
                gen_prompt = _ids(self.tok, messages[:i], tools=tools, add_generation_prompt=True) if i > 0 else []
            cur = _ids(self.tok, messages[: i + 1], tools=tools, add_generation_prompt=False)
            new = cur[len(prev):]
            if m["role"] == "assistant":
                header = max(0, len(gen_prompt) - len(prev))       # "<|im_start|>assistant\n" is context, not target
                mask += [0] * header + [1] * (len(new) - header)
            else:
                mask += [0] * len(new)
            ids += new
            prev = cur
        return ids, mask

    def __getitem__(self, i):
        r = self.rows[i]
        ids, mask = self._tokenize(r["messages"], r.get("tools"))
        L = self.max_length
        if len(ids) > L:
            if self.truncation == "error":
                raise ValueError(f"sample {i} has {len(ids)} tokens > max_length {L}")
            ids, mask = (ids[:L], mask[:L]) if self.truncation == "right" else (ids[-L:], mask[-L:])
        n = len(ids)
        pad = getattr(self.tok, "pad_token_id", 0) or 0
        input_ids = torch.full((L,), pad, dtype=torch.int64)
        att = torch.zeros(L, dtype=torch.int64)
        loss_mask = torch.zeros(L, dtype=torch.int64)
        input_ids[:n] = torch.tensor(ids)
        att[:n] = 1
        loss_mask[:n] = torch.tensor(mask)
        # the model predicts token t+1 at position t: shift so loss_mask[t] marks positions whose NEXT token is a target
        shifted = torch.zeros_like(loss_mask)
        shifted[:-1] = loss_mask[1:]
        return {"input_ids": input_ids, "attention_mask": att, "position_ids": compute_position_id_with_mask(att), "loss_mask": shifted}


class RMDataset(Dataset):
    def __init__(self, files=None, tokenizer=None, max_length: int = 512, prompt_key: str = "prompt", chosen_key: str = "chosen",
                 rejected_key: str = "rejected", rows: Optional[list] = None):
        self.tok, self.max_length = tokenizer, max_length
        if rows is None:
            df = _read(files)
            rows = [{"prompt": r[prompt_key], "chosen": r[chosen_key], "rejected": r[rejected_key]} for _, r in df.iterrows()]
        self.rows = rows

    def __len__(self):
        return len(self.rows)

    def _encode(self, prompt: str, answer: str):
        ids = self.tok.encode(prompt + answer)[: self.max_length - 1] + [self.tok.eos_token_id]
        pad = getattr(self.tok, "pad_token_id", 0) or 0
        out = torch.full((self.max_length,), pad, dtype=torch.int64)
        att = torch.zeros(self.max_length, dtype=torch.int64)
        out[: len(ids)] = torch.tensor(ids)
        att[: len(ids)] = 1
        return out, att

    def __getitem__(self, i):
        r = self.rows[i]
        c, ca = self._encode(r["prompt"], r["chosen"])
        j, ja = self._encode(r["prompt"], r["rejected"])
        return {"input_ids": torch.stack([c, j]), "attention_mask": torch.stack([ca, ja])}
