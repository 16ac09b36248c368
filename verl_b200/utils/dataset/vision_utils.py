"""Image inputs of the vision-language family: loading, the resize rule, patch extraction and placeholder expansion.

``image_to_patches`` produces what the vision tower consumes — ``pixel_values`` ``[t·h·w, C·T_p·P·P]`` with the patches of one
merge window adjacent, and ``image_grid_thw`` — without a Hugging Face processor; ``expand_image_tokens`` turns every single
image placeholder of a tokenised prompt into as many placeholders as the image has merged patches.

Reference: ``verl/utils/dataset/vision_utils.py:26-118`` (``process_image`` / ``process_video`` on top of ``qwen_vl_utils``) and
the processor call in ``verl/utils/dataset/rl_dataset.py:300-360``. Videos are taken as sequences of frames (arrays, PIL images, paths): no
container decoding happens here.
"""

from __future__ import annotations

import io
import math
from typing import Optional, Sequence

import numpy as np
import torch

__all__ = ["smart_resize", "process_image", "image_to_patches", "expand_image_tokens", "process_video", "video_to_patches", "expand_visual_tokens"]

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


def process_video(video, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280, factor: int = 28, temporal_patch_size: int = 2,
                  nframes: Optional[int] = None, fps: Optional[float] = None, max_frames: int = 768):
    """``video``: a sequence of frames (PIL images, arrays [H, W, 3], paths or bytes), an array [T, H, W, 3], or a dict
    ``{"frames" | "video": ..., "fps": source_fps, "nframes": n, "min_pixels", "max_pixels"}`` → ``(frames, seconds_per_grid_t)``:
    RGB PIL frames of one common :func:`smart_resize` size whose count is a multiple of ``temporal_patch_size`` (the last frame is
    repeated), and the time one temporal patch spans (``temporal_patch_size / sampling_fps``; 1.0 when no rate is known).
    ``nframes`` keeps that many evenly spaced frames; ``fps`` (with a known source rate) samples at that rate."""
    src_fps = None
    if isinstance(video, dict):
        min_pixels, max_pixels = video.get("min_pixels", min_pixels), video.get("max_pixels", max_pixels)
        src_fps, nframes = video.get("fps", None), video.get("nframes", nframes)
        video = video.get("frames", video.get("video"))
    frames = list(video) if not isinstance(video, (np.ndarray, torch.Tensor)) else [f for f in np.asarray(video)]
    if not frames:
        raise ValueError("a video needs at least one frame")
    T = len(frames)
    sample_fps = src_fps
    if nframes:
        keep = np.linspace(0, T - 1, int(nframes)).round().astype(int)
        sample_fps = src_fps * len(keep) / T if src_fps else None
        frames = [frames[i] for i in keep]
    elif fps and src_fps:
        n = int(min(max(round(T / src_fps * fps), temporal_patch_size), max_frames))
        keep = np.linspace(0, T - 1, n).round().astype(int)
        sample_fps, frames = float(fps), [frames[i] for i in keep]
    first = process_image(frames[0], min_pixels, max_pixels, factor)
    out = [first]
    from PIL import Image

    for f in frames[1:]:
        img = process_image(f, min_pixels, max_pixels, factor)
        out.append(img if img.size == first.size else img.resize(first.size, resample=Image.BICUBIC))
    while len(out) % temporal_patch_size:
        out.append(out[-1])
    return out, (float(temporal_patch_size) / float(sample_fps) if sample_fps else 1.0)


def video_to_patches(frames, patch_size: int = 14, temporal_patch_size: int = 2, merge_size: int = 2) -> tuple[torch.Tensor, torch.Tensor]:
    """Frames of one size (count a multiple of ``temporal_patch_size``) → (``pixel_values`` [t·h·w, 3·T_p·P·P] fp32,
    ``video_grid_thw`` [1, 3]) in the same patch order as :func:`image_to_patches`, one temporal patch after the other."""
    x = np.stack([np.asarray(f, dtype=np.float32) / 255.0 for f in frames])          # [T, H, W, 3]
    x = (x - np.asarray(IMAGE_MEAN, np.float32)) / np.asarray(IMAGE_STD, np.float32)
    x = x.transpose(0, 3, 1, 2)                                                       # [T, 3, H, W]
    T, C, H, W = x.shape
    P, m, Tp = patch_size, merge_size, temporal_patch_size
    assert T % Tp == 0 and H % (P * m) == 0 and W % (P * m) == 0, f"{T} frames of {H}x{W}"
    t, gh, gw = T // Tp, H // P, W // P
    x = x.reshape(t, Tp, C, gh // m, m, P, gw // m, m, P).transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return torch.from_numpy(np.ascontiguousarray(x.reshape(t * gh * gw, C * Tp * P * P))), torch.tensor([[t, gh, gw]])


def expand_visual_tokens(input_ids: Sequence[int], grids: torch.Tensor, token_ids: Sequence[int], merge_size: int = 2) -> list[int]:
    """Like :func:`expand_image_tokens` for prompts that mix placeholder kinds (image and video tokens): the k-th placeholder of ANY of
    ``token_ids`` is expanded to the k-th grid, so ``grids`` lists images and videos in the order they appear in the prompt."""
    out, k = [], 0
    g = grids.tolist() if grids is not None else []
    ids = set(int(t) for t in token_ids)
    for tok in input_ids:
        if tok in ids and k < len(g):
            t, h, w = g[k]
            out.extend([tok] * (t * h * w // merge_size ** 2))
            k += 1
        else:
            out.append(tok)
    assert k == len(g), f"{len(g)} visual inputs but {k} placeholders in the prompt"
    return out
