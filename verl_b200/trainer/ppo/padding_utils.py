"""Pad a global batch with dummy samples so that it divides the data-parallel size after filtering
(reference: ``verl/trainer/ppo/padding_utils.py:46-151``). Dummy rows have all masks zero, so they contribute nothing to
losses or token counts; ``is_padding`` marks them for metrics and for removal."""

from __future__ import annotations

import numpy as np
import torch

from verl_b200.protocol import DataProto, TensorBatch

__all__ = ["construct_minimal_padding_template", "upsample_batch_to_divisible_size", "remove_padding_samples"]

_MASK_KEYS = ("attention_mask", "response_mask", "loss_mask")


def construct_minimal_padding_template(batch: DataProto) -> DataProto:
    """One row shaped like the batch's rows: a single attended prompt token, everything else masked out."""
    row = batch[0:1]
    t = {}
    for k, v in row.batch.items():
        v = v.clone()
        if k in _MASK_KEYS or k.endswith("_mask"):
            v.zero_()
        elif v.dtype.is_floating_point:
            v.zero_()
        t[k] = v
    if "attention_mask" in t and "responses" in t:
        P = t["attention_mask"].shape[1] - t["responses"].shape[1]
        t["attention_mask"][:, P - 1] = 1          # keep one real token so packing never sees an empty sequence
    if "position_ids" in t:
        t["position_ids"].zero_()
    nt = {k: v.copy() for k, v in row.non_tensor_batch.items()}
    return DataProto(batch=TensorBatch(t, batch_size=(1,)), non_tensor_batch=nt, meta_info=dict(batch.meta_info))


def upsample_batch_to_divisible_size(batch: DataProto, divisor: int) -> tuple[DataProto, int]:
    n = len(batch)
    pad = (-n) % divisor
    flag = np.zeros(n + pad, dtype=bool)
    if pad == 0:
        batch.non_tensor_batch["is_padding"] = flag
        return batch, 0
    tmpl = construct_minimal_padding_template(batch)
    if "uid" in tmpl.non_tensor_batch:
        tmpl.non_tensor_batch["uid"] = np.array(["__padding__"], dtype=object)
    out = DataProto.concat([batch] + [tmpl] * pad)
    flag[n:] = True
    out.non_tensor_batch["is_padding"] = flag
    return out, pad


def remove_padding_samples(batch: DataProto) -> DataProto:
    flag = batch.non_tensor_batch.get("is_padding")
    if flag is None or not flag.any():
        return batch
    keep = torch.from_numpy(np.nonzero(~flag.astype(bool))[0])
    return batch[keep]
