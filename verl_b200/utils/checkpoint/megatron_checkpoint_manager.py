"""Checkpoints of the tensor/pipeline/data-parallel engine in the reference's Megatron "v2" directory layout
(``verl/utils/checkpoint/megatron_checkpoint_manager.py:112``, ``verl/utils/megatron_utils.py:783-895``):

    model/dist_ckpt/shard_tp{t}_pp{p}_dp{d}.pt      slice d of the flat parameter buffer of model-parallel rank (t, p)
    model/huggingface/                              config.json (+ tokenizer files, + safetensors when ``hf_model`` is saved)
    optimizer/dist_ckpt/shard_tp{t}_pp{p}_dp{d}.pt  fp32 master slice, Adam moments, step counter
    extra/dist_ckpt/shard_tp{t}_pp{p}_dp{d}.pt      LR-schedule position + RNG states
    transformer_config.json                         parallel sizes, layer ranges and the full model config
    ckpt_contents.json                              what this checkpoint holds

The distributed-checkpoint library of the reference is replaced by plain per-rank files: a rank's slice is contiguous in
its flat buffer, so one ``torch.save`` per rank is already the sharded format. Sharded files reload at the same
(tp, pp, dp); ``python -m verl_b200.model_merger merge --backend megatron`` rebuilds parallelism-independent HF weights.
"""

from __future__ import annotations

import dataclasses
import json
import os
from typing import Optional

import torch
import torch.distributed as dist

from .checkpoint_manager import BaseCheckpointManager

__all__ = ["MegatronCheckpointManager", "shard_file"]


def shard_file(root: str, part: str, tp_rank: int, pp_rank: int, dp_rank: int) -> str:
    return os.path.join(root, part, "dist_ckpt", f"shard_tp{tp_rank}_pp{pp_rank}_dp{dp_rank}.pt")


class MegatronCheckpointManager(BaseCheckpointManager):
    def __init__(self, engine, checkpoint_config=None):
        super().__init__(checkpoint_config)
        self.engine = engine

    def _files(self, root: str):
        e = self.engine
        return tuple(shard_file(root, part, e.tp_rank, e.pp_rank, e.fsdp_rank) for part in ("model", "optimizer", "extra"))

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None):
        if local_path is None:
            return
        e = self.engine
        self.previous_global_step = global_step
        if e.rank == 0:
            self.ensure_checkpoint_capacity(max_ckpt_to_keep)
            for part in ("model", "optimizer", "extra"):
                os.makedirs(os.path.join(local_path, part, "dist_ckpt"), exist_ok=True)
        if dist.is_initialized():
            dist.barrier()
        model_f, optim_f, extra_f = self._files(local_path)
        s = e.store
        contents = []
        if self.should_save_model:
            contents.append("model")
            torch.save({"format": "flat_mp_v1", "names": s.names, "shapes": [tuple(p.shape) for p in s.params], "offsets": s.offsets,
                        "total": s.total, "shard_size": s.shard_size, "dtype": str(s.flat.dtype),
                        "tp_rank": e.tp_rank, "pp_rank": e.pp_rank, "dp_rank": e.fsdp_rank, "layer_offset": getattr(e.model, "layer_offset", 0),
                        # names in the full model (under virtual pipeline stages a rank holds several layer blocks)
                        "global_names": [e._gname(n) for n in s.names] if hasattr(e, "_gname") else None,
                        "flat_shard": s.flat[s.shard_slice].detach().to("cpu", copy=True)}, model_f)
        if self.should_save_optimizer and not e.forward_only:
            contents.append("optimizer")
            torch.save({"master": e.master.detach().to("cpu", copy=True), "exp_avg": e.exp_avg.detach().to("cpu", copy=True),
                        "exp_avg_sq": e.exp_avg_sq.detach().to("cpu", copy=True), "step_count": e.step_count}, optim_f)
        if self.should_save_extra:
            contents.append("extra")
            torch.save({"lr_scheduler": {"sched_step": e.sched_step}, "rng": self.get_rng_state()}, extra_f)
        hf_tensors = None
        if self.should_save_hf_model:
            contents.append("hf_model")
            hf_tensors = list(e._gathered_hf_tensors())       # collective: every rank walks the export
        if e.rank == 0:
            hf_dir = os.path.join(local_path, "model", "huggingface")
            e.cfg.save_pretrained(hf_dir)
            tok_src = getattr(e, "tokenizer_path", None)
            if tok_src and os.path.isdir(tok_src):
                import shutil

                for fn in os.listdir(tok_src):
                    if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json", "generation_config.json"):
                        shutil.copy(os.path.join(tok_src, fn), os.path.join(hf_dir, fn))
            if hf_tensors is not None:
                from verl_b200.models.hf_io import save_hf_weights

                save_hf_weights(iter(hf_tensors), hf_dir)
            from verl_b200.models.parallel_model import stage_layer_range

            with open(os.path.join(local_path, "transformer_config.json"), "w") as f:
                json.dump({"format": "flat_mp_v1", "tensor_model_parallel_size": e.tp_size, "pipeline_model_parallel_size": e.pp_size,
                           # the weights / optimizer state of a (tp, pp) position are cut over the DP x CP ranks: that many shard files
                           "data_parallel_size": e.fsdp_size, "context_parallel_size": int(getattr(e, "cp_size", 1)), "sequence_parallel": bool(getattr(e, "tp_sp", False)),
                           "virtual_pipeline_model_parallel_size": int(getattr(e, "vpp", 1)),
                           "stage_layers": [[r.start, r.stop] for r in (stage_layer_range(e.cfg.num_hidden_layers, e.pp_size, p) for p in range(e.pp_size))],
                           "model_config": dataclasses.asdict(e.cfg) if dataclasses.is_dataclass(e.cfg) else dict(vars(e.cfg))}, f, indent=2, default=str)
            with open(os.path.join(local_path, "ckpt_contents.json"), "w") as f:
                json.dump({"contents": contents, "global_step": global_step}, f, indent=2)
        if dist.is_initialized():
            dist.barrier()
        if e.rank == 0:
            self.register_checkpoint(local_path, max_ckpt_to_keep)

    def load_checkpoint(self, local_path: Optional[str], hdfs_path: Optional[str] = None, del_local_after_load: bool = False):
        if local_path is None:
            return
        e = self.engine
        model_f, optim_f, extra_f = self._files(local_path)
        s = e.store
        tc = os.path.join(local_path, "transformer_config.json")
        if os.path.exists(tc):
            with open(tc) as f:
                meta = json.load(f)
            got = (meta["tensor_model_parallel_size"], meta["pipeline_model_parallel_size"], meta["data_parallel_size"])
            if got != (e.tp_size, e.pp_size, e.fsdp_size):
                raise ValueError(f"checkpoint was written with (tp, pp, dp x cp) = {got}, this run uses {(e.tp_size, e.pp_size, e.fsdp_size)}; "
                                 "merge it to HF weights (python -m verl_b200.model_merger merge --backend megatron) and load those")
        if self.should_load_model:
            if not os.path.exists(model_f):
                raise FileNotFoundError(model_f)
            st = torch.load(model_f, map_location="cpu", weights_only=False)
            assert st["total"] == s.total and st["names"] == s.names, "checkpoint layout does not match this model-parallel rank"
            s.flat[s.shard_slice].copy_(st["flat_shard"].to(s.flat.dtype))
            if e.fsdp_size > 1:
                if s.flat.is_cuda:
                    dist.all_gather_into_tensor(s.flat, s.flat[s.shard_slice].clone(), group=e.fsdp_group)
                else:
                    parts = [torch.empty(s.shard_size, dtype=s.flat.dtype) for _ in range(e.fsdp_size)]
                    dist.all_gather(parts, s.flat[s.shard_slice].clone(), group=e.fsdp_group)
                    s.flat.copy_(torch.cat(parts))
        optimizer_loaded = False
        if self.should_load_optimizer and not e.forward_only and os.path.exists(optim_f):
            st = torch.load(optim_f, map_location="cpu", weights_only=False)
            e.master.copy_(st["master"])
            e.exp_avg.copy_(st["exp_avg"])
            e.exp_avg_sq.copy_(st["exp_avg_sq"])
            e.step_count = int(st["step_count"])
            optimizer_loaded = True
        if self.should_load_model and not optimizer_loaded and not e.forward_only and getattr(e, "master", None) is not None:
            # weights without optimizer state: re-derive the fp32 master slice from the loaded weights and restart Adam
            e.master.copy_(s.flat[s.shard_slice].float())
            e.exp_avg.zero_()
            e.exp_avg_sq.zero_()
            e.step_count = 0
        if self.should_load_extra and os.path.exists(extra_f):
            st = torch.load(extra_f, map_location="cpu", weights_only=False)
            e.sched_step = int(st["lr_scheduler"]["sched_step"])
            self.load_rng_state(st["rng"])
        if dist.is_initialized():
            dist.barrier()
        if del_local_after_load:
            self.remove_previous_save_local_path(local_path)
