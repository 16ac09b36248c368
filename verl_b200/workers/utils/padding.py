"""Conversions between the trainer's padded layout (prompt left-padded, response right-padded) and the packed
(jagged) layout the engines consume.

Parity target: ``verl/workers/utils/padding.py`` (left_right_2_no_padding :23, no_padding_2_padding :97).
"""

from __future__ import annotations

import torch

from verl_b200.protocol import Jagged, TensorBatch

__all__ = ["left_right_2_no_padding", "no_padding_2_padding", "response_gather_index"]


def left_right_2_no_padding(batch: TensorBatch) -> TensorBatch:
    """Adds jagged ``input_ids`` / ``position_ids`` / ``loss_mask`` entries (suffix ``_packed``) built from the valid
    tokens of each row. ``loss_mask`` is 0 on prompt tokens and ``response_mask`` on response tokens."""
    ids = batch["input_ids"]
    att = batch["attention_mask"].bool()
    pos = batch["position_ids"]
    R = batch["responses"].shape[1]
    lens = att.sum(-1)
    offsets = torch.zeros(ids.shape[0] + 1, dtype=torch.int64, device=ids.device)
    offsets[1:] = torch.cumsum(lens, 0)
    resp_mask = batch["response_mask"] if "response_mask" in batch else batch["attention_mask"][:, -R:]
    full_loss = torch.cat([torch.zeros_like(batch["attention_mask"][:, :-R]), resp_mask.to(batch["attention_mask"].dtype)], dim=1)
    out = TensorBatch(batch.to_dict(), batch_size=batch.batch_size)
    out["input_ids_packed"] = Jagged(ids[att], offsets)
    out["position_ids_packed"] = Jagged(pos[att] if pos.dim() == 2 else pos[att], offsets)
    out["loss_mask_packed"] = Jagged(full_loss[att], offsets)
    return out


def response_gather_index(attention_mask: torch.Tensor, response_length: int):
    """Index into the packed token axis of the model-output position that *predicts* each response token.

    For sample i with ``p`` valid prompt tokens and ``r`` valid response tokens packed at offset ``o``, response token
    t is predicted at packed position ``o + p − 1 + t``. Returns (index [bs, R] int64, valid [bs, R] bool).
    """
    att = attention_mask.bool()
    R = response_length
    lens = att.sum(-1)
    p_len = att[:, :-R].sum(-1)
    r_len = att[:, -R:].sum(-1)
    offsets = torch.cumsum(lens, 0) - lens
    t = torch.arange(R, device=att.device)[None, :]
    idx = offsets[:, None] + p_len[:, None] - 1 + t
    valid = t < r_len[:, None]
    idx = torch.where(valid, idx, torch.zeros_like(idx))
    return idx, valid


def no_padding_2_padding(packed_values: torch.Tensor, batch: TensorBatch, pad_value: float = 0.0) -> torch.Tensor:
    """Slice per-token model outputs (packed ``[T]``) back into the right-padded response window ``[bs, R]``."""
    R = batch["responses"].shape[1]
    idx, valid = response_gather_index(batch["attention_mask"], R)
    out = packed_values[idx.reshape(-1)].reshape(idx.shape)
    return torch.where(valid, out, torch.full_like(out, pad_value))
