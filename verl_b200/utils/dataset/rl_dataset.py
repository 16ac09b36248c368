"""Prompt datasets for RL training.

* :class:`RLHFDataset` — parquet/json rows with a chat ``prompt`` column, tokenised with the model's chat template,
  left-padded to ``max_prompt_length`` (reference: ``verl/utils/dataset/rl_dataset.py:72-570``).
* :class:`SyntheticPromptDataset` — random token-id prompts of a given length range (benchmark / plumbing configs).
"""

from __future__ import annotations

import copy
import os
from typing import Optional

import numpy as np
import torch
from torch.utils.data import Dataset, RandomSampler, SequentialSampler

from verl_b200.protocol import collate_fn  # noqa: F401
from verl_b200.utils import torch_functional as VF

__all__ = ["RLHFDataset", "SyntheticPromptDataset", "collate_fn", "create_rl_dataset", "create_rl_sampler"]


def _g(cfg, key, default=None):
    v = cfg.get(key, default) if hasattr(cfg, "get") else getattr(cfg, key, default)
    return default if v is None else v


class SyntheticPromptDataset(Dataset):
    def __init__(self, num_prompts: int, min_len: int, max_len: int, id_low: int, id_high: int, max_prompt_length: int,
                 pad_token_id: int = 0, seed: int = 0, data_source: str = "synthetic/mod7"):
        g = torch.Generator().manual_seed(seed)
        self.lens = torch.randint(min_len, max_len + 1, (num_prompts,), generator=g)
        self.ids = [torch.randint(id_low, id_high, (int(n),), generator=g) for n in self.lens]
        self.max_prompt_length = max_prompt_length
        self.pad = pad_token_id
        self.data_source = data_source

    def __len__(self):
        return len(self.ids)

    def __getitem__(self, i):
        ids = self.ids[i]
        P = self.max_prompt_length
        n = ids.numel()
        input_ids = torch.full((P,), self.pad, dtype=torch.int64)
        att = torch.zeros(P, dtype=torch.int64)
        input_ids[P - n:] = ids
        att[P - n:] = 1
        return {"input_ids": input_ids, "attention_mask": att, "position_ids": VF.compute_position_id_with_mask(att),
                "data_source": self.data_source, "reward_model": {"style": "rule", "ground_truth": int(ids.sum()) % 7},
                "index": i, "extra_info": {"index": i}}


class RLHFDataset(Dataset):
    def __init__(self, data_files, tokenizer, config, processor=None, max_samples: int = -1):
        import pandas as pd

        self.tokenizer = tokenizer
        self.config = config
        files = [data_files] if isinstance(data_files, str) else list(data_files)
        frames = []
        for f in files:
            f = os.path.expanduser(f)
            frames.append(pd.read_parquet(f) if f.endswith(".parquet") else pd.read_json(f, lines=f.endswith(".jsonl")))
        self.df = pd.concat(frames, ignore_index=True)
        if max_samples and max_samples > 0:
            self.df = self.df.iloc[:max_samples]
        self.prompt_key = _g(config, "prompt_key", "prompt")
        self.max_prompt_length = int(_g(config, "max_prompt_length", 1024))
        self.truncation = _g(config, "truncation", "error")
        self.return_raw_chat = bool(_g(config, "return_raw_chat", True))
        self.return_full_prompt = bool(_g(config, "return_full_prompt", False))
        self.apply_chat_template_kwargs = dict(_g(config, "apply_chat_template_kwargs", {}) or {})
        # vision-language prompts: column with the images of a row and the tower geometry (VisionConfig fields)
        self.image_key = _g(config, "image_key", "images")
        self.video_key = _g(config, "video_key", "videos")           # per row: a list of videos, each a sequence of frames
        self.vision = dict(_g(config, "vision", None) or {}) or None
        if bool(_g(config, "filter_overlong_prompts", False)):
            keep = [len(self._tokenize(self._messages(row))) <= self.max_prompt_length for _, row in self.df.iterrows()]
            self.df = self.df[np.asarray(keep)].reset_index(drop=True)

    def _messages(self, row):
        msgs = row[self.prompt_key]
        if isinstance(msgs, np.ndarray):
            msgs = msgs.tolist()
        if isinstance(msgs, str):
            msgs = [{"role": "user", "content": msgs}]
        return [dict(m) for m in msgs]

    def _tokenize(self, messages):
        if getattr(self.tokenizer, "chat_template", None):
            text = self.tokenizer.apply_chat_template(messages, add_generation_prompt=True, tokenize=False, **self.apply_chat_template_kwargs)
        else:
            text = "\n".join(m["content"] for m in messages)
        if self.vision and ("<image>" in text or "<video>" in text) and "<|image_pad|>" not in text and "<|video_pad|>" not in text:
            # a tokenizer whose chat template knows nothing about images: every "<image>" / "<video>" mark becomes
            # vision_start, ONE placeholder of its kind (expanded to the input's size later), vision_end
            import re

            v = self.vision
            vs = int(v.get("vision_start_token_id", 151652))
            ve = int(v.get("vision_end_token_id", vs + 1))
            marks = {"<image>": [vs, int(v.get("image_token_id", 151655)), ve], "<video>": [vs, int(v.get("video_token_id", 151656)), ve]}
            ids = []
            for part in re.split(r"(<image>|<video>)", text):
                if part in marks:
                    ids += marks[part]
                elif part:
                    ids += self.tokenizer(part, add_special_tokens=False)["input_ids"]
            return ids
        return self.tokenizer(text, add_special_tokens=False)["input_ids"]

    def _with_images(self, tok_ids, images, videos=()):
        """Patches of the row's images and videos and the prompt with every placeholder expanded to its input's merged patches.
        Patches and grids are kept in the order the placeholders appear in the prompt (images and videos interleaved), which is the
        order the tower's output rows are matched to the placeholder tokens in; ``grid_t_scale`` holds, per grid, the factor the
        temporal positions of a video advance by per temporal patch (seconds per patch x the model's tokens per second; 1 for images)."""
        from verl_b200.utils.dataset.vision_utils import expand_visual_tokens, image_to_patches, process_image, process_video, video_to_patches

        v = self.vision
        P, Tp, m = int(v.get("patch_size", 14)), int(v.get("temporal_patch_size", 2)), int(v.get("spatial_merge_size", 2))
        lo = int(_g(self.config, "image_min_pixels", None) or 4 * (P * m) ** 2)
        hi = int(_g(self.config, "image_max_pixels", None) or 1280 * (P * m) ** 2)
        img_id, vid_id = int(v.get("image_token_id", 151655)), int(v.get("video_token_id", 151656))
        images, videos = list(images), list(videos)
        pix, grids, scales = [], [], []
        for tok in tok_ids:
            if tok == img_id and images:
                p, g = image_to_patches(process_image(images.pop(0), factor=P * m, min_pixels=lo, max_pixels=hi), P, Tp, m)
                sc = 1.0
            elif tok == vid_id and videos:
                frames, sec = process_video(videos.pop(0), min_pixels=int(_g(self.config, "video_min_pixels", None) or lo),
                                            max_pixels=int(_g(self.config, "video_max_pixels", None) or hi), factor=P * m, temporal_patch_size=Tp,
                                            nframes=_g(self.config, "video_nframes", None), fps=_g(self.config, "video_fps", None))
                p, g = video_to_patches(frames, P, Tp, m)
                sc = sec * float(v.get("tokens_per_second", 0) or 0) if v.get("tokens_per_second") else 1.0
            else:
                continue
            pix.append(p)
            grids.append(g)
            scales.append(sc)
        assert not images and not videos, "more images / videos in the row than placeholders in the prompt"
        grids = torch.cat(grids, 0)
        tok_ids = expand_visual_tokens(tok_ids, grids, (img_id, vid_id), m)
        mm = {"pixel_values": torch.cat(pix, 0), "image_grid_thw": grids}
        if any(s_ != 1.0 for s_ in scales):
            mm["grid_t_scale"] = torch.tensor(scales, dtype=torch.float32)
        return tok_ids, mm

    def __len__(self):
        return len(self.df)

    def __getitem__(self, i):
        row = self.df.iloc[i].to_dict()
        messages = self._messages(row)
        tok_ids = self._tokenize(messages)
        images = row.get(self.image_key) if self.vision else None
        videos = row.get(self.video_key) if self.vision else None
        mm = None
        if (images is not None and len(images)) or (videos is not None and len(videos)):
            tok_ids, mm = self._with_images(tok_ids, list(images) if images is not None else [], list(videos) if videos is not None else [])
        ids = torch.tensor(tok_ids, dtype=torch.int64)[None]
        att = torch.ones_like(ids)
        pad = self.tokenizer.pad_token_id if self.tokenizer.pad_token_id is not None else 0
        ids, att = VF.postprocess_data(ids, att, self.max_prompt_length, pad, left_pad=True, truncation="error" if mm else self.truncation)
        out = {k: v for k, v in row.items() if k not in (self.prompt_key,) + ((self.image_key, self.video_key) if self.vision else ())}
        out.update({"input_ids": ids[0], "attention_mask": att[0], "position_ids": VF.compute_position_id_with_mask(att[0])})
        if self.vision:
            # [4, L]: text positions first, then the temporal / height / width streams of the multimodal rotary embedding
            from verl_b200.models.vision import VisionConfig, get_rope_index

            vcfg = VisionConfig(**{**self.vision, "mrope_section": tuple(self.vision.get("mrope_section", (16, 24, 24)))})
            pos3, _ = get_rope_index(ids[0], mm["image_grid_thw"] if mm else None, vcfg, attention_mask=att[0], grid_t_scale=mm.get("grid_t_scale") if mm else None)
            out["position_ids"] = torch.cat([out["position_ids"][None], pos3], 0)
            out["multi_modal_inputs"] = mm or {}
        if self.return_raw_chat:
            out["raw_prompt"] = messages
        extra = out.get("extra_info") or {}
        out["index"] = extra.get("index", i) if isinstance(extra, dict) else i
        out.setdefault("data_source", "unknown")
        return out

    def resume_dataset_state(self):
        pass


def create_rl_dataset(data_files, data_config, tokenizer, processor=None, is_train: bool = True, max_samples: int = -1):
    syn = _g(data_config, "synthetic", None)
    if syn is not None and _g(syn, "enable", False):
        return SyntheticPromptDataset(int(_g(syn, "num_prompts", 4096)), int(_g(syn, "min_prompt_length", 16)), int(_g(syn, "max_prompt_length", 32)),
                                      int(_g(syn, "id_low", 10)), int(_g(syn, "id_high", 2048)), int(_g(data_config, "max_prompt_length", 512)),
                                      seed=int(_g(data_config, "seed", 0)) + (0 if is_train else 1))
    custom = _g(data_config, "custom_cls", None)
    if custom is not None and _g(custom, "path", None):
        from verl_b200.utils.import_utils import load_extern_type

        cls = load_extern_type(custom["path"], custom["name"])
        return cls(data_files=data_files, tokenizer=tokenizer, config=data_config, processor=processor)
    return RLHFDataset(data_files, tokenizer, data_config, processor, max_samples)


def create_rl_sampler(data_config, dataset):
    if bool(_g(data_config, "shuffle", True)):
        g = torch.Generator()
        g.manual_seed(int(_g(data_config, "seed", 1)))
        return RandomSampler(dataset, generator=g)
    return SequentialSampler(dataset)
