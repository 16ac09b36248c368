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
                 truncation: str = "right", rows: Optional[list] = None, vision: Optional[dict] = None, images_key: str = "images",
                 image_min_pixels: Optional[int] = None, image_max_pixels: Optional[int] = None):
        """``vision`` (fields of ``verl_b200.models.vision.VisionConfig``) switches image support on: a row's ``images`` are cut
        into patches, every ``<image>`` mark (or image placeholder token written by the chat template) is expanded to the
        image's merged patches, and the item carries ``multi_modal_inputs`` and 4-stream ``position_ids``."""
        assert truncation in ("right", "left", "error")
        self.tok, self.max_length, self.truncation = tokenizer, max_length, truncation
        self.vision, self.image_pixels = (dict(vision) if vision else None), (image_min_pixels, image_max_pixels)
        if rows is None:
            df = _read(files)
            rows = [{"messages": list(r[messages_key]), "tools": (list(r[tools_key]) if tools_key in df.columns and r[tools_key] is not None else None),
                     "images": (list(r[images_key]) if images_key in df.columns and r[images_key] is not None else None)}
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

    def _with_images(self, ids: list, mask: list, images: list):
        from verl_b200.utils.dataset.vision_utils import image_to_patches, process_image

        v = self.vision
        P, Tp, m = int(v.get("patch_size", 14)), int(v.get("temporal_patch_size", 2)), int(v.get("spatial_merge_size", 2))
        img_id, vs = int(v.get("image_token_id", 151655)), int(v.get("vision_start_token_id", 151652))
        if img_id not in ids:              # plain-text "<image>" marks: vision_start, one placeholder, vision_end
            mark = self.tok("<image>", add_special_tokens=False)["input_ids"]
            out_i, out_m, j = [], [], 0
            while j < len(ids):
                if ids[j:j + len(mark)] == mark:
                    out_i += [vs, img_id, int(v.get("vision_end_token_id", vs + 1))]
                    out_m += [0, 0, 0]
                    j += len(mark)
                else:
                    out_i.append(ids[j])
                    out_m.append(mask[j])
                    j += 1
            ids, mask = out_i, out_m
        pix, grids = [], []
        for img in images:
            p, g = image_to_patches(process_image(img, factor=P * m, min_pixels=int(self.image_pixels[0] or 4 * (P * m) ** 2),
                                                  max_pixels=int(self.image_pixels[1] or 1280 * (P * m) ** 2)), P, Tp, m)
            pix.append(p)
            grids.append(g)
        grids = torch.cat(grids, 0)
        out_i, out_m, k = [], [], 0
        for t, mk in zip(ids, mask):
            if t == img_id and k < len(grids):
                n = int(grids[k, 0] * grids[k, 1] * grids[k, 2]) // (m * m)
                out_i += [img_id] * n
                out_m += [0] * n
                k += 1
            else:
                out_i.append(t)
                out_m.append(mk)
        assert k == len(grids), f"{len(grids)} images but {k} image placeholders in the conversation"
        return out_i, out_m, {"pixel_values": torch.cat(pix, 0), "image_grid_thw": grids}

    def __getitem__(self, i):
        r = self.rows[i]
        ids, mask = self._tokenize(r["messages"], r.get("tools"))
        mm = None
        if self.vision and r.get("images"):
            ids, mask, mm = self._with_images(ids, mask, list(r["images"]))
            if len(ids) > self.max_length:
                raise ValueError(f"sample {i} has {len(ids)} tokens with its images expanded > max_length {self.max_length} (images are never truncated)")
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
        item = {"input_ids": input_ids, "attention_mask": att, "position_ids": compute_position_id_with_mask(att), "loss_mask": shifted}
        if self.vision:
            from verl_b200.models.vision import VisionConfig, get_rope_index

            vcfg = VisionConfig(**{**self.vision, "mrope_section": tuple(self.vision.get("mrope_section", (16, 24, 24)))})
            pos3, _ = get_rope_index(input_ids, mm["image_grid_thw"] if mm else None, vcfg, attention_mask=att)
            item["position_ids"] = torch.cat([item["position_ids"][None], pos3], 0)
            item["multi_modal_inputs"] = mm or {}
        return item


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
