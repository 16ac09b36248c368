"""Image inputs of the vision-language family: loading, the resize rule, patch extraction and placeholder expansion.

``image_to_patches`` produces what the vision tower consumes — ``pixel_values`` ``[t·h·w, C·T_p·P·P]`` with the patches of one
merge window adjacent, and ``image_grid_thw`` — without a Hugging Face processor; ``expand_image_tokens`` turns every single
image placeholder of a tokenised prompt into as many placeholders as the image has merged patches.

Reference: ``verl/utils/dataset/vision_utils.py:26-118`` (``process_image`` / ``process_video`` on top of ``qwen_vl_utils``) and
the processor call in ``verl/utils/dataset/rl_dataset.py:300-360``. Video inputs are not supported.
"""

from __future__ import annotations

import io
import math
from typing import Sequence

import numpy as np
import torch

__all__ = ["smart_resize", "process_image", "image_to_patches", "expand_image_tokens", "process_video"]

IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[int, int]:
    """Target size: both sides multiples of ``factor`` (patch × merge), area within [min_pixels, max_pixels], aspect kept."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError(f"aspect ratio of a {height}x{width} image is above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def process_image(image, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280, factor: int = 28):
    """``image``: a PIL image, a path, raw bytes, or a dict with one of ``image`` / ``bytes`` / ``path`` (the parquet layouts
    of image datasets) and optional ``min_pixels`` / ``max_pixels`` → an RGB PIL image of the :func:`smart_resize` size."""
    from PIL import Image

    if isinstance(image, dict):
        min_pixels, max_pixels = image.get("min_pixels", min_pixels), image.get("max_pixels", max_pixels)
        image = image.get("image", image.get("bytes", image.get("path")))
    if isinstance(image, (bytes, bytearray)):
        image = Image.open(io.BytesIO(image))
    elif isinstance(image, str):
        image = Image.open(image)
    elif isinstance(image, (np.ndarray, torch.Tensor)):
        image = Image.fromarray(np.asarray(image).astype(np.uint8))
    image = image.convert("RGB")
    h, w = smart_resize(image.height, image.width, factor, min_pixels, max_pixels)
    return image.resize((w, h), resample=Image.BICUBIC) if (h, w) != (image.height, image.width) else image


def image_to_patches(image, patch_size: int = 14, temporal_patch_size: int = 2, merge_size: int = 2) -> tuple[torch.Tensor, torch.Tensor]:
    """A resized RGB image (sides multiples of ``patch_size · merge_size``) → (``pixel_values`` [h·w, 3·T_p·P·P] fp32,
    ``image_grid_thw`` [1, 3]). A still image is repeated along time to fill one temporal patch."""
    x = np.asarray(image, dtype=np.float32) / 255.0                       # [H, W, 3]
    x = (x - np.asarray(IMAGE_MEAN, np.float32)) / np.asarray(IMAGE_STD, np.float32)
    x = x.transpose(2, 0, 1)[None].repeat(temporal_patch_size, 0)          # [T_p, 3, H, W]
    C, H, W = x.shape[1:]
    P, m = patch_size, merge_size
    assert H % (P * m) == 0 and W % (P * m) == 0, f"{H}x{W} is not a multiple of {P * m}"
    gh, gw = H // P, W // P
    x = x.reshape(1, temporal_patch_size, C, gh // m, m, P, gw // m, m, P).transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return torch.from_numpy(np.ascontiguousarray(x.reshape(gh * gw, C * temporal_patch_size * P * P))), torch.tensor([[1, gh, gw]])


def expand_image_tokens(input_ids: Sequence[int], grids: torch.Tensor, image_token_id: int, merge_size: int = 2) -> list[int]:
    """Replace the k-th image placeholder by ``t·h·w / merge²`` placeholders (the number of rows the tower returns for it)."""
    out, k = [], 0
    g = grids.tolist() if grids is not None else []
    for tok in input_ids:
        if tok == image_token_id and k < len(g):
            t, h, w = g[k]
            out.extend([image_token_id] * (t * h * w // merge_size ** 2))
            k += 1
        else:
            out.append(tok)
    assert k == len(g), f"{len(g)} images but {k} image placeholders in the prompt"
    return out


def process_video(video, **kwargs):
    raise NotImplementedError("video inputs are not supported by the vision-language family of this framework")
