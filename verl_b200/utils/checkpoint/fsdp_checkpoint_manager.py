"""Per-rank sharded checkpoints of the fsdp engine.

Directory layout (same file names as the reference, ``verl/utils/checkpoint/fsdp_checkpoint_manager.py:364-527``):

    model_world_size_{W}_rank_{r}.pt        this rank's slice of the flat parameter buffer + layout table
    optim_world_size_{W}_rank_{r}.pt        fp32 master slice, Adam moments, step counters
    extra_state_world_size_{W}_rank_{r}.pt  LR-schedule position + RNG states (cpu / numpy / random / cuda)
    fsdp_config.json                        {"FSDP_version": 2, "world_size": W, "format": "flat_v1"}
    huggingface/                            config.json (+ safetensors shards when ``hf_model`` is in save_contents)

Only same-world-size reloads are supported for the ``flat_v1`` sharded files (as in the reference); ``huggingface/`` and
``python -m verl_b200.model_merger`` give the world-size-independent form.

Interchange with the reference's payload (``checkpoint.model_format: dtensor``): the model file then holds ``{HF name:
DTensor}`` with dim-0 shards exactly as the reference writes it, so its loader and merger read it; on load the format is detected
from the file, and a checkpoint written by the reference (any world size) is merged and loaded as weights
(``dtensor_interchange.py``).
"""

from __future__ import annotations

import json
import os
import threading
from typing import Optional

import torch
import torch.distributed as dist

from .checkpoint_manager import ASYNC_PENDING, BaseCheckpointManager

__all__ = ["FSDPCheckpointManager"]


class FSDPCheckpointManager(BaseCheckpointManager):
    def __init__(self, engine, checkpoint_config=None):
        super().__init__(checkpoint_config)
        self.engine = engine
        self._async_thread: Optional[threading.Thread] = None
        cfg = checkpoint_config or {}
        fmt = cfg.get("model_format", None) if hasattr(cfg, "get") else getattr(cfg, "model_format", None)
        self.model_format = str(fmt or "flat_v1")
        if self.model_format not in ("flat_v1", "dtensor"):
            raise ValueError(f"checkpoint.model_format must be flat_v1 or dtensor, got {self.model_format!r}")

    @property
    def rank(self):
        return self.engine.fsdp_rank + self.engine.fsdp_size * (self.engine.rank // self.engine.fsdp_size)

    def _names(self, local_path):
        W, r = self.engine.world, self.engine.rank
        return (os.path.join(local_path, f"model_world_size_{W}_rank_{r}.pt"),
                os.path.join(local_path, f"optim_world_size_{W}_rank_{r}.pt"),
                os.path.join(local_path, f"extra_state_world_size_{W}_rank_{r}.pt"))

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None):
        if local_path is None:
            return
        e = self.engine
        self.previous_global_step = global_step
        self.wait_async_save()
        if dist.is_initialized():
            dist.barrier()                      # every rank's previous writer is done: older checkpoints may go
        if e.rank == 0:
            # while background writers run, the newest complete checkpoint must survive: keep one more than asked for
            keep = max_ckpt_to_keep + 1 if self.async_save and isinstance(max_ckpt_to_keep, int) and max_ckpt_to_keep > 0 else max_ckpt_to_keep
            self.ensure_checkpoint_capacity(keep)
            self.local_mkdir_safe(local_path)
            if self.async_save:
                with open(os.path.join(local_path, ASYNC_PENDING), "w") as f:
                    f.write(str(e.world))
        self.local_mkdir_safe(local_path)
        if dist.is_initialized():
            dist.barrier()
        model_f, optim_f, extra_f = self._names(local_path)
        s = e.store
        payload = []
        zero3_now = bool(getattr(e, "_zero3_rows", None))
        if self.should_save_model and self.model_format == "dtensor":
            from .dtensor_interchange import dtensor_model_payload

            if zero3_now or getattr(e.model, "lora_config", None):
                raise NotImplementedError("checkpoint.model_format=dtensor is available for full resident weights (no ZeRO-3 row sharding, no LoRA adapters)")
            payload.append((model_f, dtensor_model_payload(e.model.hf_named_tensors(), e.rank, e.world, e.fsdp_size)))
        elif self.should_save_model:
            shard = s.flat[s.shard_slice].detach().to("cpu", copy=True)
            payload.append((model_f, {"format": "flat_v1", "names": s.names, "shapes": [tuple(p.shape) for p in s.params],
                                      "offsets": s.offsets, "total": s.total, "shard_size": s.shard_size,
                                      "fsdp_rank": e.fsdp_rank, "fsdp_size": e.fsdp_size, "dtype": str(s.flat.dtype),
                                      "zero3_rows": dict(getattr(e, "_zero3_rows", None) or {}), "rank": e.rank, "world": e.world,
                                      "flat_shard": shard}))
        if self.should_save_optimizer and not e.forward_only:
            payload.append((optim_f, {"master": e.master.detach().to("cpu", copy=True), "exp_avg": e.exp_avg.detach().to("cpu", copy=True),
                                      "exp_avg_sq": e.exp_avg_sq.detach().to("cpu", copy=True), "step_count": e.step_count}))
        if self.should_save_extra:
            payload.append((extra_f, {"lr_scheduler": {"sched_step": e.sched_step}, "rng": self.get_rng_state()}))

        marker = self.async_marker(local_path, e.rank) if self.async_save else None

        def write():
            for fn, obj in payload:
                tmp = fn + ".tmp"
                torch.save(obj, tmp)
                os.replace(tmp, fn)
            if marker is not None:
                open(marker, "w").close()       # this rank's files are complete

        if self.async_save:
            self._async_thread = threading.Thread(target=write, daemon=True)
            self._async_thread.start()
        else:
            write()
        zero3 = bool(getattr(e, "_zero3_rows", None))
        if e.rank == 0:
            with open(os.path.join(local_path, "fsdp_config.json"), "w") as f:
                meta = {"FSDP_version": 2, "world_size": e.world, "format": self.model_format}
                if getattr(e.model, "lora_config", None):
                    meta["lora"] = dict(e.model.lora_config)       # the shards then hold the adapters only (python -m verl_b200.scripts.merge_lora)
                json.dump(meta, f, indent=2)
            hf_dir = os.path.join(local_path, "huggingface")
            e.cfg.save_pretrained(hf_dir)
            tok_src = getattr(e, "tokenizer_path", None)
            if tok_src and os.path.isdir(tok_src):
                import shutil
                for fn in os.listdir(tok_src):
                    if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json", "generation_config.json"):
                        shutil.copy(os.path.join(tok_src, fn), os.path.join(hf_dir, fn))
            if self.should_save_hf_model and not zero3:
                from verl_b200.models.hf_io import save_hf_weights

                save_hf_weights(e.model.hf_named_tensors(), hf_dir)
        if self.should_save_hf_model and zero3:
            # row-sharded weights: the export gathers them one by one, a collective that every rank walks through
            it = e.hf_named_tensors_for_save()
            if e.rank == 0:
                from verl_b200.models.hf_io import save_hf_weights

                save_hf_weights(it, os.path.join(local_path, "huggingface"))
            else:
                for _ in it:
                    pass
        if dist.is_initialized():
            dist.barrier()
        if e.rank == 0:
            self.register_checkpoint(local_path, max_ckpt_to_keep)

    def load_checkpoint(self, local_path: Optional[str], hdfs_path: Optional[str] = None, del_local_after_load: bool = False):
        if local_path is None:
            return
        e = self.engine
        model_f, optim_f, extra_f = self._names(local_path)
        s = e.store
        named_format = False
        if self.should_load_model:
            from .dtensor_interchange import is_named_tensor_payload, merge_sharded_model_files, saved_world_size

            probe = model_f if os.path.exists(model_f) else None
            if probe is None:       # another world size: only the named-tensor form can be re-cut
                try:
                    probe = os.path.join(local_path, f"model_world_size_{saved_world_size(local_path)}_rank_0.pt")
                except FileNotFoundError:
                    probe = None
            if probe is None or not os.path.exists(probe):
                raise FileNotFoundError(f"{model_f} not found (flat_v1 sharded checkpoints reload only at the same world size)")
            st = torch.load(probe, map_location="cpu", weights_only=False)
            named_format = is_named_tensor_payload(st)
            if not named_format and probe != model_f:
                raise FileNotFoundError(f"{model_f} not found (flat_v1 sharded checkpoints reload only at the same world size)")
        if self.should_load_model and named_format:
            # the reference's payload: every rank merges the dim-0 shards and copies the weights into its resident parameters
            del st
            e.model.load_hf_state_dict(merge_sharded_model_files(local_path), strict=True)
        elif self.should_load_model:
            assert st["total"] == s.total and st["names"] == s.names, "checkpoint layout does not match this model"
            s.flat[s.shard_slice].copy_(st["flat_shard"].to(s.flat.dtype))
            if e.world > 1 and e.fsdp_size > 1:
                if s.flat.is_cuda:
                    dist.all_gather_into_tensor(s.flat, s.flat[s.shard_slice].clone(), group=e.fsdp_group)
                else:
                    parts = [torch.empty(s.shard_size, dtype=s.flat.dtype) for _ in range(e.fsdp_size)]
                    dist.all_gather(parts, s.flat[s.shard_slice].clone(), group=e.fsdp_group)
                    s.flat.copy_(torch.cat(parts))
        optimizer_loaded = False
        if self.should_load_optimizer and not e.forward_only and os.path.exists(optim_f) and not named_format:
            st = torch.load(optim_f, map_location="cpu", weights_only=False)
            if "master" not in st:
                raise ValueError(f"{optim_f} holds per-parameter optimizer state of another framework; set checkpoint.load_contents=[model] to load the weights only")
            e.master.copy_(st["master"])
            e.exp_avg.copy_(st["exp_avg"])
            e.exp_avg_sq.copy_(st["exp_avg_sq"])
            e.step_count = int(st["step_count"])
            optimizer_loaded = True
        if self.should_load_model and not optimizer_loaded and not e.forward_only and getattr(e, "master", None) is not None:
            # weights without optimizer state: the fp32 master copy must follow the loaded weights, otherwise the next
            # optimizer step would write the initialisation-time master (plus one update) over them
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
