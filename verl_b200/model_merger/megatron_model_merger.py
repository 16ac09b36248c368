"""Merge a checkpoint of the tensor/pipeline/data-parallel engine (``model/dist_ckpt/shard_tp*_pp*_dp*.pt``) into HF weights.

For every model-parallel rank (t, p) the data-parallel slices are concatenated back into that rank's flat buffer and cut into
its local tensors; local layer indices are shifted by the stage's layer offset; tensor-parallel pieces are joined along
their split dimension (fused qkv / gate_up are joined per segment); the result goes through the native→HF name mapping.
Parity target: ``verl/model_merger/megatron_model_merger.py:37-108`` (which rebuilds an mcore model and exports through a
bridge; here the layout table stored with each shard is enough).
"""

from __future__ import annotations

import json
import os
from concurrent.futures import ThreadPoolExecutor

import torch

from .base_model_merger import BaseModelMerger

__all__ = ["MegatronModelMerger"]


class MegatronModelMerger(BaseModelMerger):
    def _meta(self) -> dict:
        path = os.path.join(self.config.local_dir, "transformer_config.json")
        if not os.path.exists(path):
            raise FileNotFoundError(f"transformer_config.json not found in {self.config.local_dir}")
        with open(path) as f:
            return json.load(f)

    def _local_tensors(self, tp_rank: int, pp_rank: int, dp: int) -> dict[str, torch.Tensor]:
        from verl_b200.models.parallel_model import local_to_global_name
        from verl_b200.utils.checkpoint.megatron_checkpoint_manager import shard_file

        shards = [torch.load(shard_file(self.config.local_dir, "model", tp_rank, pp_rank, d), map_location="cpu", weights_only=False)
                  for d in range(dp)]
        first = shards[0]
        if first.get("format") != "flat_mp_v1":
            raise ValueError("unsupported shard format (expected flat_mp_v1)")
        flat = torch.cat([s["flat_shard"] for s in shards])
        assert flat.numel() >= first["total"], "data-parallel slices do not add up to the recorded buffer length"
        out = {}
        gnames = first.get("global_names") or [local_to_global_name(name, int(first["layer_offset"])) for name in first["names"]]
        for name, shape, off in zip(gnames, first["shapes"], first["offsets"]):
            n = 1
            for d in shape:
                n *= d
            out[name] = flat[off: off + n].view(*shape)
        return out

    def _merge(self) -> dict[str, torch.Tensor]:
        from verl_b200.models.parallel_model import unshard_param
        from verl_b200.models.transformer import native_to_hf_tensors

        meta = self._meta()
        tp, pp, dp = int(meta["tensor_model_parallel_size"]), int(meta["pipeline_model_parallel_size"]), int(meta["data_parallel_size"])
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
            loaded = list(ex.map(lambda tp_pp: self._local_tensors(tp_pp[0], tp_pp[1], dp), [(t, p) for p in range(pp) for t in range(tp)]))
        native: dict[str, torch.Tensor] = {}
        for p in range(pp):
            per_tp = loaded[p * tp: (p + 1) * tp]
            for name in per_tp[0]:
                if name in native:      # tied embedding kept on the first and the last stage: identical copies
                    continue
                native[name] = unshard_param(name, [d[name] for d in per_tp], self.model_config)
        return {k: v.to(torch.bfloat16).clone() for k, v in native_to_hf_tensors(self.model_config, native)}

    def merge_and_save(self):
        sd = self._merge()
        if self.config.operation == "test":
            if not self.config.test_hf_dir:
                raise ValueError("test_hf_dir must be provided for test operation")
            self._validate_against_hf(sd)
        elif self.config.operation == "merge":
            self.save_hf_model_and_tokenizer(sd)
            if self.config.hf_upload:
                self.upload_to_huggingface()
        else:
            raise ValueError(f"Unknown operation: {self.config.operation}")

    def cleanup(self):
        pass
