"""Sharded data-parallel training engine ("fsdp" backend).

Design for a 180 GB B200: the bf16 working copy of the parameters is one flat buffer that stays *resident* on every
rank (ZeRO-2 style, ``reshard_after_forward=False``) while fp32 master weights, Adam moments and the reduced
gradients are sharded 1/W per rank. One optimizer step is: reduce-scatter(fp32 grads) → global-norm clip → fused
AdamW on the local shard (writes the bf16 shard) → all-gather of the bf16 shards. Compared with the reference's
per-layer all-gather/reduce-scatter on every micro-batch (``verl/workers/engine/fsdp/transformer_impl.py:389-498``,
``verl/utils/fsdp_utils.py:549-614``) this removes all collectives from forward/backward and lets the colocated
rollout engine read the same resident weights with no copy. ``reshard_after_forward=True`` (ZeRO-3) keeps only the
shard resident and gathers layer units on demand.

Parity target for behaviour: ``FSDPEngine`` in ``verl/workers/engine/fsdp/transformer_impl.py`` (forward_backward_batch
:728-781, optimizer_step :792-838, prepare_model_inputs/outputs :1155-1568, get_per_tensor_param :981-1065).
"""

from __future__ import annotations

import math
import os
from contextlib import contextmanager
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from verl_b200 import ops
from verl_b200.models.config import PRESETS, ModelConfig
from verl_b200.models.transformer import DecoderLM, PackedBatch
from verl_b200.ops import _ext
from verl_b200.utils.device import get_device_name
from verl_b200.utils.metric import AggregationType, Metric
from verl_b200.utils.seqlen_balancing import rearrange_micro_batches, restore_dynamic_batch
from verl_b200.workers.engine.base import BaseEngine, EngineRegistry
from verl_b200.workers.utils.padding import response_gather_index

__all__ = ["FSDPEngine", "FSDPEngineWithValueHead", "FlatParamStore", "cfg_get"]


def cfg_get(cfg, key: str, default=None):
    """Read ``a.b.c`` from nested dict-likes / dataclasses, returning ``default`` for missing or None values."""
    cur = cfg
    for part in key.split("."):
        if cur is None:
            return default
        if hasattr(cur, "get") and not isinstance(cur, torch.Tensor):
            cur = cur.get(part, None)
        else:
            cur = getattr(cur, part, None)
    return default if cur is None else cur


# bytes moved host->device (inputs, from pinned memory) and device->host (results) by the engines of this process
IO_STATS = {"h2d_bytes": 0, "d2h_bytes": 0}


def _to_device(v: torch.Tensor, dev: torch.device) -> torch.Tensor:
    if v.device == dev:
        return v
    if dev.type == "cuda" and v.device.type == "cpu":
        IO_STATS["h2d_bytes"] += v.numel() * v.element_size()
        return v.pin_memory().to(dev, non_blocking=True)
    return v.to(dev)


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "float16": torch.float16, "fp16": torch.float16, "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}


class FlatParamStore:
    """All parameters of a model as views into one flat buffer (+ a flat fp32 gradient buffer of the same layout).

    Every tensor starts on a 256-byte boundary so each view is a legal TMA base; the total length is padded so it
    divides evenly among ``world`` ranks in 1024-element granules.
    """

    ALIGN = 128

    def __init__(self, model: torch.nn.Module, world: int, rank: int, order_key=None):
        self.model = model
        self.world, self.rank = world, rank
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]   # frozen tensors (LoRA base) stay outside
        if order_key is not None:
            params.sort(key=order_key)                                              # stable: model order within equal keys
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += -(-p.numel() // self.ALIGN) * self.ALIGN
        gran = world * 1024
        self.total = -(-off // gran) * gran
        self.shard_size = self.total // world
        dev, dt = self.params[0].device, self.params[0].dtype
        self.flat = torch.zeros(self.total, dtype=dt, device=dev)
        for p, o in zip(self.params, self.offsets):
            view = self.flat[o : o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
        self.grad: Optional[torch.Tensor] = None

    @property
    def shard_slice(self) -> slice:
        return slice(self.rank * self.shard_size, (self.rank + 1) * self.shard_size)

    def alloc_grads(self):
        if self.grad is None:
            self.grad = torch.zeros(self.total, dtype=torch.float32, device=self.flat.device)
            for p, o in zip(self.params, self.offsets):
                p.main_grad = self.grad[o : o + p.numel()].view(p.shape)

    def free_grads(self):
        self.grad = None
        for p in self.params:
            p.main_grad = None

    def zero_grads(self):
        if self.grad is not None:
            self.grad.zero_()
        for p in self.params:
            p.grad = None

    def fold_autograd_grads(self):
        """Parameters touched by plain PyTorch ops receive ``.grad``; add those into the flat buffer."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None

    def rebind(self, new_flat: torch.Tensor):
        """Point every parameter at ``new_flat`` (same layout) — used by offload and symmetric-heap placement."""
        self.flat = new_flat
        for p, o in zip(self.params, self.offsets):
            p.data = new_flat[o : o + p.numel()].view(p.shape)


def _adamw_reference(p32, m, v, g, lr, b1, b2, eps, wd, step, gscale):
    """torch.optim.AdamW update rule (decoupled weight decay) on flat fp32 tensors."""
    g = g.float() * gscale
    p32.mul_(1 - lr * wd)
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    bc1 = 1 - b1**step
    bc2 = 1 - b2**step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p32.addcdiv_(m, denom, value=-lr / bc1)


@EngineRegistry.register(model_type="language_model", backend=["fsdp", "fsdp2"], device=["cuda", "cpu"])
class FSDPEngine(BaseEngine):
    def __init__(self, model_config, engine_config=None, optimizer_config=None, checkpoint_config=None):
        self.model_config = model_config
        self.engine_config = engine_config or {}
        self.optimizer_config = optimizer_config
        self.checkpoint_config = checkpoint_config or {}
        self.mode = None
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.device = torch.device(get_device_name(), torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.sp_size = int(cfg_get(self.engine_config, "ulysses_sequence_parallel_size", 1) or 1)
        # context parallelism shares the sequence-parallel plumbing (token slicing, output gather, gradient scaling); only
        # attention differs: K/V are all-gathered instead of scattering heads (verl_b200.parallel.context_parallel)
        cp = int(cfg_get(self.engine_config, "context_parallel_size", 1) or 1)
        self.sp_mode = "ulysses"
        if cp > 1:
            assert self.sp_size == 1, "choose either ulysses_sequence_parallel_size or context_parallel_size"
            self.sp_size, self.sp_mode = cp, "context"
        # zig-zag placement of the context-parallel slices balances the causal attention work between the ranks
        self._cp_zigzag = self.sp_mode == "context" and bool(cfg_get(self.engine_config, "context_parallel_zigzag", False))
        # dynamic context parallelism: per micro-batch every sample gets the smallest aligned sub-group of the CP ranks that keeps
        # its share under ``max_seqlen_per_dp_cp_rank`` (short samples run on one rank without any communication)
        self._dynamic_cp = self.sp_mode == "context" and bool(cfg_get(self.engine_config, "dynamic_context_parallel", False))
        if self._dynamic_cp:
            assert self.sp_size & (self.sp_size - 1) == 0, "dynamic context parallelism needs a power-of-two context_parallel_size"
        fsdp_size = int(cfg_get(self.engine_config, "fsdp_size", -1))
        self.fsdp_size = self.world if fsdp_size in (-1, 0) or fsdp_size >= self.world else fsdp_size
        self.forward_only = bool(cfg_get(self.engine_config, "forward_only", False)) or optimizer_config is None
        self._param_offload = bool(cfg_get(self.engine_config, "param_offload", False))
        self._optimizer_offload = bool(cfg_get(self.engine_config, "optimizer_offload", False))
        self.step_count = 0
        self.sched_step = 0
        self._value_head = False
        self.model: Optional[DecoderLM] = None
        self.store: Optional[FlatParamStore] = None

    # ------------------------------------------------------------------ build
    def _resolve_model_config(self) -> ModelConfig:
        mc = self.model_config
        if isinstance(mc, ModelConfig):
            cfg = mc
        else:
            preset = cfg_get(mc, "preset", None)
            path = cfg_get(mc, "path", None)
            if preset is not None:
                cfg = PRESETS[preset]
            elif path is not None and os.path.exists(os.path.join(os.path.expanduser(path), "config.json")):
                cfg = ModelConfig.from_pretrained(os.path.expanduser(path))
            elif path in PRESETS:
                cfg = PRESETS[path]
            else:
                raise FileNotFoundError(f"cannot resolve model config from {mc}")
            override = cfg_get(mc, "override_config", None) or {}
            override = {k: v for k, v in dict(override).items() if k in ModelConfig.__dataclass_fields__}
            if override:
                cfg = cfg.replace(**override)
        if self._value_head and not cfg.value_head:
            cfg = cfg.replace(value_head=True)
        return cfg

    def initialize(self):
        cfg = self._resolve_model_config()
        self.cfg = cfg
        dt_name = cfg_get(self.engine_config, "model_dtype", None) or (cfg.torch_dtype if self.device.type == "cpu" else "bfloat16")
        self.dtype = _DTYPES.get(str(dt_name), torch.bfloat16)
        seed = int(cfg_get(self.engine_config, "seed", 0))
        if cfg.vision:
            # vision-language family: tower + decoder behind the decoder's interface (verl_b200.models.vision)
            from verl_b200.models.vision import VisionLanguageModel

            assert self.sp_size == 1, "vision-language models do not run under sequence/context parallelism yet"
            self.model = VisionLanguageModel(cfg, dtype=self.dtype, device=self.device, init=True, seed=seed)
        else:
            self.model = DecoderLM(cfg, dtype=self.dtype, device=self.device, init=True, seed=seed)
        path = cfg_get(self.model_config, "path", None) if not isinstance(self.model_config, ModelConfig) else None
        if path and os.path.isdir(os.path.expanduser(path)):
            from verl_b200.models.hf_io import load_hf_weights

            load_hf_weights(self.model, os.path.expanduser(path), strict=not cfg.value_head)
        self.model.gradient_checkpointing = bool(cfg_get(self.model_config, "enable_gradient_checkpointing", False))
        if not isinstance(self.model_config, ModelConfig) and bool(cfg_get(self.model_config, "enable_activation_offload", False)) \
                and self.device.type == "cuda" and not self.forward_only:
            # tensors saved for backward inside the decoder layers wait in pinned host memory (copied on a side stream, prefetched
            # one layer ahead in backward)
            from verl_b200.utils.activation_offload import enable_activation_offloading

            enable_activation_offloading(self.model, int(cfg_get(self.model_config, "activation_offload_min_numel", 1 << 20)))
        tiled = cfg_get(self.model_config, "tiled_mlp", None) if not isinstance(self.model_config, ModelConfig) else None
        if tiled is not None and bool(cfg_get(tiled, "enabled", False)):
            for layer in self.model.layers:
                if hasattr(layer.mlp, "tiled_shards"):
                    layer.mlp.tiled_shards = int(cfg_get(tiled, "num_shards", 4))
        lora_rank = int(cfg_get(self.model_config, "lora_rank", 0) or 0) if not isinstance(self.model_config, ModelConfig) else 0
        if lora_rank > 0 and not self.forward_only:
            from verl_b200.models.lora import apply_lora

            apply_lora(self.model, lora_rank, float(cfg_get(self.model_config, "lora_alpha", 2 * lora_rank)),
                       cfg_get(self.model_config, "target_modules", "all-linear"), seed=seed)
        self._build_groups()
        self._place_parameters()
        if self.sp_size > 1:
            self.model.sp_group = self.sp_group
            from verl_b200.parallel.ulysses import FusedUlysses, fused_ulysses_available

            for layer in self.model.layers:
                layer.self_attn.sp_mode = self.sp_mode
            probe = self.store.flat[:1]
            if self.sp_mode == "ulysses" and fused_ulysses_available(probe, cfg, self.sp_size) and bool(cfg_get(self.engine_config, "fused_ulysses", True)):
                from verl_b200.single_controller.spmd import init_spmd_process_group

                init_spmd_process_group()
                max_tok = int(cfg_get(self.engine_config, "ulysses_max_tokens", 65536))
                self._fused_ulysses = FusedUlysses(self.sp_group, self._sp_host_group(), cfg, max_tok)
                for layer in self.model.layers:
                    layer.self_attn.fused_ulysses = self._fused_ulysses
        if not self.forward_only:
            self._build_optimizer()
        from verl_b200.utils.checkpoint.fsdp_checkpoint_manager import FSDPCheckpointManager

        self.checkpoint_manager = FSDPCheckpointManager(self, self.checkpoint_config)
        if self._param_offload:
            self.to("cpu", model=True, optimizer=False, grad=False)
        if self._optimizer_offload and not self.forward_only:
            self.to("cpu", model=False, optimizer=True, grad=True)

    def _place_parameters(self):
        """Lay the parameters out in the flat store (replicated working copy; symmetric memory when the fused optimizer applies)."""
        self.store = FlatParamStore(self.model, self.fsdp_size, self.fsdp_rank)
        if self.world > 1:
            # every rank must start from identical weights (rank 0's)
            dist.broadcast(self.store.flat, src=0)
        self._symm_params = self._symm_grads = None
        use_symm = bool(cfg_get(self.engine_config, "use_symmetric_memory", True)) and os.environ.get("VERL_B200_COMM", "native") == "native"
        if (use_symm and self.world > 1 and self.fsdp_size == self.world and self.store.flat.is_cuda and self.store.flat.dtype == torch.bfloat16
                and _ext.available() and not self.forward_only and not self._param_offload):
            from verl_b200.parallel.symm_mem import SymmetricBuffer
            from verl_b200.single_controller.spmd import init_spmd_process_group

            host = init_spmd_process_group()
            s = self.store
            self._symm_params = SymmetricBuffer(s.total * 2, host_group=host)
            new_flat = self._symm_params.tensor(torch.bfloat16, s.total)
            new_flat.copy_(s.flat)
            s.rebind(new_flat)
            self._symm_grads = SymmetricBuffer(s.total * 4, host_group=host)

    def _build_groups(self):
        """Mesh (ddp, fsdp) for parameter sharding and (dp, sp) for Ulysses; ranks are laid out fsdp/sp-fastest."""
        self.fsdp_group = self.ddp_group = self.sp_group = self.dp_group = None
        self.fsdp_rank, self.ddp_size = self.rank % self.fsdp_size, self.world // self.fsdp_size
        self.sp_rank = self.rank % self.sp_size
        self.dp_size = self.world // self.sp_size
        self.dp_rank = self.rank // self.sp_size
        if self.world == 1:
            return
        if self.fsdp_size == self.world:
            self.fsdp_group = dist.group.WORLD
        else:
            for d in range(self.ddp_size):
                ranks = list(range(d * self.fsdp_size, (d + 1) * self.fsdp_size))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.fsdp_group = g
            for f in range(self.fsdp_size):
                ranks = list(range(f, self.world, self.fsdp_size))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.ddp_group = g
        if self.sp_size > 1:
            assert self.world % self.sp_size == 0
            for d in range(self.dp_size):
                ranks = list(range(d * self.sp_size, (d + 1) * self.sp_size))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.sp_group = g
            for s in range(self.sp_size):
                ranks = list(range(s, self.world, self.sp_size))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.dp_group = g
            self._dcp_groups = {}
            if getattr(self, "_dynamic_cp", False):
                # aligned sub-groups of every width below the full one: width k -> the group this rank belongs to
                k = 2
                while k < self.sp_size:
                    for d in range(self.dp_size):
                        for start in range(0, self.sp_size, k):
                            ranks = [d * self.sp_size + start + i for i in range(k)]
                            g = dist.new_group(ranks)
                            if self.rank in ranks:
                                self._dcp_groups[k] = g
                    k *= 2
                self._dcp_groups[self.sp_size] = self.sp_group
        else:
            self.dp_group = dist.group.WORLD

    def _sp_host_group(self):
        """gloo twin of the SP group (pointer-table exchange of the symmetric buffers goes through host memory)."""
        if getattr(self, "_sp_host", None) is None:
            mine = None
            for d in range(self.dp_size):
                ranks = list(range(d * self.sp_size, (d + 1) * self.sp_size))
                g = dist.new_group(ranks, backend="gloo")
                if self.rank in ranks:
                    mine = g
            self._sp_host = mine
        return self._sp_host

    def _build_optimizer(self):
        oc = self.optimizer_config
        self.lr = float(cfg_get(oc, "lr", 1e-6))
        betas = cfg_get(oc, "betas", (0.9, 0.999))
        self.beta1, self.beta2 = float(betas[0]), float(betas[1])
        self.adam_eps = float(cfg_get(oc, "eps", 1e-8))
        self.weight_decay = float(cfg_get(oc, "weight_decay", 0.01))
        self.clip_grad = float(cfg_get(oc, "clip_grad", 1.0))
        self.total_steps = int(cfg_get(oc, "total_training_steps", -1))
        warm = int(cfg_get(oc, "lr_warmup_steps", -1))
        if warm < 0:
            ratio = float(cfg_get(oc, "lr_warmup_steps_ratio", 0.0))
            warm = int(ratio * max(self.total_steps, 0))
        self.warmup_steps = warm
        self.lr_scheduler_type = cfg_get(oc, "lr_scheduler_type", cfg_get(oc, "warmup_style", "constant"))
        self.min_lr_ratio = float(cfg_get(oc, "min_lr_ratio", 0.0))
        self.num_cycles = float(cfg_get(oc, "num_cycles", 0.5))
        s = self.store
        shard = s.flat[s.shard_slice]
        self.master = shard.detach().clone().float()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_shard = None
        self._scalars = torch.zeros(4, dtype=torch.float32, device=self.device)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)

    def current_lr(self) -> float:
        step = self.sched_step
        if self.warmup_steps > 0 and step < self.warmup_steps:
            return self.lr * step / max(1, self.warmup_steps)
        if self.lr_scheduler_type == "cosine" and self.total_steps > 0:
            prog = (step - self.warmup_steps) / max(1, self.total_steps - self.warmup_steps)
            coef, icpt = (1 - self.min_lr_ratio) * 0.5, (1 + self.min_lr_ratio) * 0.5
            return self.lr * max(self.min_lr_ratio, math.cos(math.pi * self.num_cycles * 2.0 * prog) * coef + icpt)
        return self.lr

    # ------------------------------------------------------------------ properties
    @property
    def is_param_offload_enabled(self) -> bool:
        return self._param_offload

    @property
    def is_optimizer_offload_enabled(self) -> bool:
        return self._optimizer_offload

    def get_data_parallel_rank(self) -> int:
        return self.dp_rank

    def get_data_parallel_size(self) -> int:
        return self.dp_size

    def get_data_parallel_group(self):
        return self.dp_group

    def is_mp_src_rank_with_outputs(self) -> bool:
        return self.sp_rank == 0

    # ------------------------------------------------------------------ placement / offload
    def to(self, device: str, model: bool = True, optimizer: bool = True, grad: bool = True):
        if self.device.type == "cpu":
            return
        target = self.device if device in ("cuda", "gpu", str(self.device)) else torch.device("cpu")
        to_cpu = target.type == "cpu"
        if model and self.store is not None:
            if to_cpu and self.store.flat.is_cuda:
                host = getattr(self, "_host_flat", None)
                if host is None or not self.forward_only:
                    host = torch.empty(self.store.flat.shape, dtype=self.store.flat.dtype, pin_memory=True)
                    host.copy_(self.store.flat, non_blocking=True)
                    torch.cuda.current_stream().synchronize()
                    IO_STATS["d2h_bytes"] += host.numel() * host.element_size()
                    if self.forward_only:
                        self._host_flat = host      # frozen weights: the pinned copy stays valid, later offloads copy nothing
                self.store.rebind(host)
            elif not to_cpu and not self.store.flat.is_cuda:
                IO_STATS["h2d_bytes"] += self.store.flat.numel() * self.store.flat.element_size()
                pre = getattr(self, "_prefetched", None)
                self._prefetched = None
                if pre is not None and pre[0].shape == self.store.flat.shape:
                    # the copy was started earlier on a side stream (prefetch_params): only wait for it
                    dev_flat, ev = pre
                    torch.cuda.current_stream().wait_event(ev)
                    dev_flat.record_stream(torch.cuda.current_stream())
                    self.store.rebind(dev_flat)
                else:
                    self.store.rebind(self.store.flat.to(target, non_blocking=True))
        if optimizer and not self.forward_only:
            for name in ("master", "exp_avg", "exp_avg_sq"):
                t = getattr(self, name)
                if to_cpu and t.is_cuda:
                    host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                    host.copy_(t, non_blocking=True)
                    setattr(self, name, host)
                elif not to_cpu and not t.is_cuda:
                    setattr(self, name, t.to(target, non_blocking=True))
            torch.cuda.current_stream().synchronize()
        if grad and to_cpu and self.store is not None:
            self.store.free_grads()
        if to_cpu:
            torch.cuda.empty_cache()

    def prefetch_params(self) -> bool:
        """Start bringing offloaded (pinned-host) parameters back on a side stream, so that the copy runs under whatever the
        GPU is doing now; the next ``to("cuda")`` only waits for it. Used for the frozen reference policy: its 2 bytes per
        parameter cross PCIe while the actor's old-log-prob pass computes. Returns True when a copy was started."""
        if self.device.type != "cuda" or self.store is None or self.store.flat.is_cuda or getattr(self, "_prefetched", None) is not None:
            return False
        if not self.store.flat.is_pinned():
            return False
        if getattr(self, "_prefetch_stream", None) is None:
            self._prefetch_stream = torch.cuda.Stream()
        with torch.cuda.stream(self._prefetch_stream):
            dev_flat = torch.empty(self.store.flat.shape, dtype=self.store.flat.dtype, device=self.device)
            dev_flat.copy_(self.store.flat, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._prefetch_stream)
        self._prefetched = (dev_flat, ev)
        return True

    # ------------------------------------------------------------------ micro-batching
    def _prefix_sharing(self, meta: dict, tensors: dict) -> bool:
        """Prefix sharing (one prompt forward for its n responses) applies to policy passes without Ulysses slicing."""
        return bool(meta.get("use_prefix_grouper", False)) and self.sp_size == 1 and not self.cfg.value_head and "responses" in tensors

    def _micro_batch_indices(self, seq_lens: torch.Tensor, meta: dict, tensors: Optional[dict] = None) -> list[list[int]]:
        n = seq_lens.numel()
        if tensors is not None and meta.get("use_dynamic_bsz", False) and self._prefix_sharing(meta, tensors):
            from verl_b200.utils.prefix_sharing import group_preserving_micro_batches, prompt_groups

            att = tensors["attention_mask"]
            P = att.shape[1] - tensors["responses"].shape[1]
            gid, _ = prompt_groups(tensors["input_ids"], att, P)
            pl, rl = att[:, :P].sum(-1).cpu(), att[:, P:].sum(-1).cpu()
            budget = int(meta["max_token_len_per_gpu"])
            parts = group_preserving_micro_batches(rl, pl, gid.cpu(), budget)
            if self.world > 1 and dist.is_initialized():
                t = torch.tensor([len(parts)], device=self.device if dist.get_backend(self.dp_group) == "nccl" else "cpu")
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.dp_group)
                parts = group_preserving_micro_batches(rl, pl, gid.cpu(), budget, num_micro_batches=int(t.item()))
            return parts
        if meta.get("use_dynamic_bsz", False):
            budget = int(meta["max_token_len_per_gpu"]) * self.sp_size
            return rearrange_micro_batches(seq_lens.cpu(), budget, dp_group=self.dp_group if self.world > 1 else None)
        mbs = int(meta.get("micro_batch_size_per_gpu", 0) or n)
        return [list(range(i, min(n, i + mbs))) for i in range(0, n, mbs)]

    def _pack(self, mb: dict) -> tuple[PackedBatch, torch.Tensor]:
        att = mb["attention_mask"].bool()
        ids = mb["input_ids"][att]
        pos_full, pos3 = mb["position_ids"], None
        if pos_full.dim() == 3:
            # multimodal rotary embedding: [bs, 3, L] (temporal, height, width) or [bs, 4, L] with the text positions first
            # (reference: verl/utils/dataset/rl_dataset.py:330-360)
            pos3 = pos_full[:, -3:].transpose(0, 1)[:, att]
            pos_full = pos_full[:, 0]
        pos = pos_full[att]
        lens = att.sum(-1)
        cu_cpu = torch.zeros(lens.numel() + 1, dtype=torch.int32)
        cu_cpu[1:] = torch.cumsum(lens.cpu(), 0)
        cu = cu_cpu.to(ids.device, non_blocking=True)
        labels = torch.roll(ids, shifts=-1, dims=0)
        routed = None
        if "routed_experts" in mb:
            routed = mb["routed_experts"][att]
        pb = PackedBatch(ids, pos.to(torch.int32), cu, cu_cpu, int(lens.max()), routed)
        mm_rows = mb.get("multi_modal_inputs")
        if mm_rows is not None or pos3 is not None:
            pb.mm = self._multi_modal(mb, mm_rows or [], pos3, att)
        return pb, labels

    def _multi_modal(self, mb: dict, rows: list, pos3, att: torch.Tensor) -> dict:
        """Image patches of the micro-batch's rows in token order, their grids and the 3-stream positions of the packed tokens
        (computed from the token ids when the batch carries plain 1-D positions)."""
        dev = att.device
        pix = [torch.as_tensor(r["pixel_values"]) for r in rows if r and r.get("pixel_values") is not None and len(r["pixel_values"])]
        grids = [torch.as_tensor(r["image_grid_thw"]).reshape(-1, 3) for r in rows if r and r.get("image_grid_thw") is not None and len(r["image_grid_thw"])]
        if pos3 is None and self.cfg.vision:
            from verl_b200.models.vision import VisionConfig, get_rope_index

            v = dict(self.cfg.vision)
            vcfg = VisionConfig(**{**v, "mrope_section": tuple(v["mrope_section"])})
            ids_cpu, att_cpu = mb["input_ids"].cpu(), att.cpu()
            per_row = []
            for i in range(ids_cpu.shape[0]):
                r = rows[i] if i < len(rows) and rows[i] else {}
                g = torch.as_tensor(r["image_grid_thw"]).reshape(-1, 3) if r.get("image_grid_thw") is not None and len(r["image_grid_thw"]) else None
                sc = torch.as_tensor(r["grid_t_scale"]) if r.get("grid_t_scale") is not None else None
                p, _ = get_rope_index(ids_cpu[i], g, vcfg, attention_mask=att_cpu[i], grid_t_scale=sc)
                per_row.append(p[:, att_cpu[i]])
            pos3 = torch.cat(per_row, 1).to(dev)
        return {"pixel_values": torch.cat(pix, 0).to(dev) if pix else None, "image_grid_thw": torch.cat(grids, 0) if grids else None,
                "mrope_positions": pos3}

    def _forward_micro_batch(self, mb: dict, meta: dict) -> dict:
        """Returns per-token outputs already sliced to the response window: tensors of shape [bs, R]."""
        pb, labels = self._pack(mb)
        R = mb["responses"].shape[1]
        idx, valid = response_gather_index(mb["attention_mask"], R)
        if pb.mm is None and self._prefix_sharing(meta, mb):
            return self._forward_shared_prefix(mb, pb, labels, idx, valid, meta)
        temperature = float(meta.get("temperature", 1.0))
        need_entropy = bool(meta.get("calculate_entropy", False))
        out: dict[str, torch.Tensor] = {}
        if self.cfg.value_head:
            vals = self.model(pb)["values"]
            out["values"] = torch.where(valid, vals[idx.reshape(-1)].reshape(idx.shape), torch.zeros((), device=vals.device))
            return out
        if self.sp_size > 1:
            lp, ent = self._sp_forward(pb, labels, temperature, need_entropy)
            full = torch.zeros(idx.shape, dtype=torch.float32, device=lp.device)
            out["log_probs"] = torch.where(valid, lp[idx.reshape(-1)].reshape(idx.shape), full)
            if ent is not None:
                out["entropy"] = torch.where(valid, ent[idx.reshape(-1)].reshape(idx.shape), full)
            return out
        record = bool(meta.get("record_routing", False)) and self.cfg.is_moe and pb.routed_experts is None
        if record:
            for layer in self.model.layers:
                layer.mlp.record_routing = True
        h = self.model.forward_hidden(pb)
        if record:
            # router replay R2: the experts this pass chose, laid out like input_ids so that the update pass can force them
            rt = torch.stack([layer.mlp.last_topk for layer in self.model.layers], 1).to(torch.int16)      # [T, layers, topk]
            att = mb["attention_mask"].bool()
            full_rt = torch.full((*att.shape, *rt.shape[1:]), -1, dtype=torch.int16, device=rt.device)
            full_rt[att] = rt
            out["routed_experts"] = full_rt
            for layer in self.model.layers:
                layer.mlp.record_routing = False
        sel = idx[valid]
        h_sel = h.index_select(0, sel)
        lp, ent = ops.linear_logprob_entropy(h_sel, self.model.output_weight, labels.index_select(0, sel), temperature, need_entropy)
        full = torch.zeros(idx.shape, dtype=torch.float32, device=h.device)
        out["log_probs"] = full.masked_scatter(valid, lp.float())
        if ent is not None:
            out["entropy"] = torch.zeros_like(full).masked_scatter(valid, ent.float())
        self._score_centering_terms(out, mb, meta, h_sel, valid, temperature)
        return out

    def _score_centering_terms(self, out: dict, mb: dict, meta: dict, h_sel: torch.Tensor, valid: torch.Tensor, temperature: float) -> None:
        """Score centering (train–inference mismatch correction): log-probs of the sampler's top-k head under the trainer,
        turned into the per-token correction term that the REINFORCE loss adds (reference:
        verl/trainer/ppo/score_centering.py:217-257). ``h_sel`` are the hidden rows that predict the valid response tokens."""
        self._distillation_terms(out, mb, meta, h_sel, valid, temperature)
        if not meta.get("score_centering", False) or "rollout_topk_ids" not in mb:
            return
        from verl_b200.trainer.ppo.score_centering import score_centering_correction, score_centering_weight_fn, topk_log_probs_from_hidden

        ids = mb["rollout_topk_ids"][valid]
        lq = mb["rollout_topk_log_probs"][valid]
        lp_head = topk_log_probs_from_hidden(h_sel, self.model.output_weight, ids, temperature)
        wfn = score_centering_weight_fn(meta.get("rollout_is", None), meta.get("rollout_is_threshold", 2.0))
        corr, q_mass, p_mass = score_centering_correction(lp_head, lq, wfn)
        zero = torch.zeros(valid.shape, dtype=torch.float32, device=h_sel.device)
        out["sc_correction"] = zero.masked_scatter(valid, corr.float())
        out["sc_sampler_head_mass"] = zero.masked_scatter(valid, q_mass.float()).detach()
        out["sc_train_head_mass"] = zero.masked_scatter(valid, p_mass.float()).detach()

    def _distillation_terms(self, out: dict, mb: dict, meta: dict, h_sel: torch.Tensor, valid: torch.Tensor, temperature: float) -> None:
        """On-policy distillation. Teacher pass (``meta["return_topk"] = k``): the k most likely next tokens and their
        log-probs at every response position. Student pass (batch holds ``teacher_topk_ids``): the student's log-probs of
        those ids, with gradient. Logits exist for 1024 rows at a time only. Reference: prompt-logprob requests to a
        teacher server, verl/experimental/teacher_loop/teacher_manager.py:36-144."""
        k = int(meta.get("return_topk", 0) or 0)
        W = self.model.output_weight
        if k > 0:
            ids, lps = [], []
            with torch.no_grad():
                for s0 in range(0, h_sel.shape[0], 1024):
                    x = ops.linear(h_sel[s0: s0 + 1024], W).float() / temperature
                    v, i = torch.log_softmax(x, -1).topk(k, -1)
                    ids.append(i)
                    lps.append(v)
            bs, R = valid.shape
            tid = torch.zeros(bs, R, k, dtype=torch.int64, device=h_sel.device)
            tlp = torch.full((bs, R, k), -1e4, dtype=torch.float32, device=h_sel.device)
            if ids:
                tid[valid] = torch.cat(ids)
                tlp[valid] = torch.cat(lps)
            out["topk_ids"], out["topk_log_probs"] = tid, tlp
        if meta.get("distillation", False) and "teacher_topk_ids" in mb:
            from verl_b200.trainer.ppo.score_centering import topk_log_probs_from_hidden

            ids = mb["teacher_topk_ids"][valid]
            lp = topk_log_probs_from_hidden(h_sel, W, ids, temperature)
            full = torch.full((*valid.shape, ids.shape[-1]), -1e4, dtype=torch.float32, device=h_sel.device)
            out["student_topk_log_probs"] = full.masked_scatter(valid[..., None].expand_as(full), lp.float())

    def _forward_shared_prefix(self, mb: dict, pb_full: PackedBatch, labels_full: torch.Tensor, idx, valid, meta: dict) -> dict:
        """Policy forward on the unique tokens of the micro-batch: every distinct prompt once plus all responses. Attention
        expands to full sequences through ``PackedBatch.attn_expand``; the rows that predict response tokens are looked up
        in the unique layout (the last prompt row serves all n first response tokens of its group)."""
        from verl_b200.utils.prefix_sharing import build_shared_pack, prompt_groups

        att = mb["attention_mask"]
        P = att.shape[1] - mb["responses"].shape[1]
        _, first_row = prompt_groups(mb["input_ids"], att, P)
        sp = build_shared_pack(att, P, first_row)
        routed = mb["routed_experts"][sp.keep] if "routed_experts" in mb else None
        pb = PackedBatch(mb["input_ids"][sp.keep], mb["position_ids"][sp.keep].to(torch.int32), pb_full.cu_seqlens, pb_full.cu_seqlens_cpu,
                         pb_full.max_seqlen, routed)
        pb.attn_expand = (sp.expand, sp.back, sp.order, sp.offsets)
        h = self.model.forward_hidden(pb)
        sel = idx[valid]
        temperature = float(meta.get("temperature", 1.0))
        need_entropy = bool(meta.get("calculate_entropy", False))
        h_sel = h.index_select(0, sp.expand.index_select(0, sel))      # a few repeats only (last prompt row of each group)
        lp, ent = ops.linear_logprob_entropy(h_sel, self.model.output_weight, labels_full.index_select(0, sel), temperature, need_entropy)
        full = torch.zeros(idx.shape, dtype=torch.float32, device=h.device)
        out = {"log_probs": full.masked_scatter(valid, lp.float())}
        if ent is not None:
            out["entropy"] = torch.zeros_like(full).masked_scatter(valid, ent.float())
        self._score_centering_terms(out, mb, meta, h_sel, valid, temperature)
        return out

    def _sp_forward(self, pb: PackedBatch, labels: torch.Tensor, temperature: float, need_entropy: bool):
        """Ulysses sequence parallelism: every rank of the SP group holds the same micro-batch, runs the model on its
        slice of the packed tokens (attention sees the whole sequences through the all-to-all) and the per-token outputs are
        gathered back; gradients are scaled so that summing over the SP ranks gives the full-batch gradient."""
        from verl_b200.parallel.ulysses import gather_outputs_and_unpad, ulysses_pad_and_slice_inputs

        sp, r = self.sp_size, self.sp_rank
        T = pb.input_ids.shape[0]
        if self._cp_zigzag:
            from verl_b200.parallel.context_parallel import zigzag_permutation

            pad = (-T) % (2 * sp)
            ids, pos, lab = pb.input_ids, pb.position_ids, labels
            if pad:
                ids, lab = torch.nn.functional.pad(ids, (0, pad)), torch.nn.functional.pad(lab, (0, pad))
                pos = torch.cat([pos, torch.arange(pad, device=pos.device, dtype=pos.dtype)])
            perm = zigzag_permutation(T + pad, sp).to(ids.device)
            Tl = (T + pad) // sp
            mine = perm[r * Tl:(r + 1) * Tl]
            pbl = PackedBatch(ids.index_select(0, mine), pos.index_select(0, mine), pb.cu_seqlens, pb.cu_seqlens_cpu, pb.max_seqlen, None)
            pbl.cp_zigzag = True
            h = self.model.forward_hidden(pbl)
            lp_l, ent_l = ops.linear_logprob_entropy(h, self.model.output_weight, lab.index_select(0, mine), temperature, need_entropy)
            inv = torch.argsort(perm)          # gathered rows come in rank order; put them back into stream order
            lp = gather_outputs_and_unpad(lp_l.float(), 0, None, 0, grad_scaler=True, group=self.sp_group).index_select(0, inv)[:T]
            ent = gather_outputs_and_unpad(ent_l.float(), 0, None, 0, grad_scaler=True, group=self.sp_group).index_select(0, inv)[:T] \
                if ent_l is not None else None
            return lp, ent
        ids_l, pos_l, pad = ulysses_pad_and_slice_inputs(pb.input_ids, pb.position_ids, sp, r, dim=0)
        lab = torch.nn.functional.pad(labels, (0, pad)) if pad else labels
        Tl = (T + pad) // sp
        lab_l = lab[r * Tl:(r + 1) * Tl]
        pbl = PackedBatch(ids_l, pos_l, pb.cu_seqlens, pb.cu_seqlens_cpu, pb.max_seqlen, None)
        gpos = pb.position_ids
        if pad:
            gpos = torch.cat([gpos, torch.arange(pad, device=gpos.device, dtype=gpos.dtype)])
        pbl.global_position_ids = gpos
        h = self.model.forward_hidden(pbl)
        lp_l, ent_l = ops.linear_logprob_entropy(h, self.model.output_weight, lab_l, temperature, need_entropy)
        lp = gather_outputs_and_unpad(lp_l.float(), 0, 0, pad, grad_scaler=True, group=self.sp_group)
        ent = gather_outputs_and_unpad(ent_l.float(), 0, 0, pad, grad_scaler=True, group=self.sp_group) if ent_l is not None else None
        return lp, ent

    # ------------------------------------------------------------------ forward / backward
    def forward_backward_batch(self, data, loss_function: Optional[Callable], forward_only: bool = False) -> dict:
        if getattr(self, "_dynamic_cp", False) and self.sp_size > 1:
            return self._forward_backward_dynamic_cp(data, loss_function, forward_only)
        batch = data.batch
        meta = dict(getattr(data, "meta_info", {}) or {})
        dev = self.device
        tensors = {k: (_to_device(v, dev) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        n = tensors["input_ids"].shape[0]
        seq_lens = tensors["attention_mask"].sum(-1)
        mb_indices = self._micro_batch_indices(seq_lens, meta, tensors)
        mm_rows = (getattr(data, "non_tensor_batch", None) or {}).get("multi_modal_inputs")      # per-row dicts (vision-language models)
        # global normalisers for the loss (identical on all ranks)
        info: dict[str, Any] = {"dp_size": self.dp_size}
        if not forward_only and loss_function is not None:
            mask_key = "response_mask" if "response_mask" in tensors else None
            ntok = tensors[mask_key].sum().to(torch.float32) if mask_key else seq_lens.sum().to(torch.float32)
            cnt = torch.stack([ntok, torch.tensor(float(n), device=dev)])
            if self.world > 1:
                dist.all_reduce(cnt, group=self.dp_group)
                if self.sp_size > 1:
                    pass  # data is replicated inside an sp group; dp_group spans one rank per sp group
            info["batch_num_tokens"] = cnt[0]
            info["global_batch_size"] = cnt[1]
            if not forward_only:
                self._alloc_grads()
        outputs: dict[str, list[torch.Tensor]] = {}
        metrics: dict[str, Metric] = {}
        losses = []
        self.model.train(not forward_only)
        for idxs in mb_indices:
            it = torch.as_tensor(idxs, device=dev)
            mb = {k: (v.index_select(0, it) if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == n else v)
                  for k, v in tensors.items()}
            if mm_rows is not None:
                mb["multi_modal_inputs"] = [mm_rows[i] for i in idxs]
            ctx = torch.no_grad() if forward_only else torch.enable_grad()
            with ctx:
                mo = self._forward_micro_batch(mb, meta)
                if loss_function is not None:
                    mb_data = dict(mb)
                    mb_data.update(info)
                    loss, m = loss_function(model_output=mo, data=mb_data, dp_group=self.dp_group)
                    if not forward_only:
                        loss.backward()
                    losses.append(float(loss.detach()))
                    for k, v in m.items():
                        if k in metrics:
                            metrics[k].append(v)
                        else:
                            metrics[k] = v if isinstance(v, Metric) else Metric(AggregationType.MEAN, v)
            for k, v in mo.items():
                outputs.setdefault(k, []).append(v.detach())
            off = getattr(self.model, "_activation_offloader", None)
            if off is not None:
                off.reset()          # the micro-batch's saved tensors have been consumed (or were never needed: forward only)
        if not forward_only and loss_function is not None:
            self.store.fold_autograd_grads()
        model_output = {k: restore_dynamic_batch(torch.cat(v, 0), mb_indices) for k, v in outputs.items()}
        return {"model_output": model_output, "loss": losses, "metrics": metrics}

    @contextmanager
    def _sub_sp(self, k: int, cp_rank: int):
        """Run the enclosed forward with a context-parallel group of width ``k`` (1 = no sequence parallelism at all)."""
        saved = (self.sp_size, self.sp_rank, self.sp_group, self.model.sp_group)
        g = None if k == 1 else self._dcp_groups[k]
        self.sp_size, self.sp_rank, self.sp_group, self.model.sp_group = k, cp_rank, g, g
        try:
            yield
        finally:
            self.sp_size, self.sp_rank, self.sp_group, self.model.sp_group = saved

    def _forward_backward_dynamic_cp(self, data, loss_function: Optional[Callable], forward_only: bool) -> dict:
        """``forward_backward_batch`` with dynamic context parallelism (reference: ``verl/utils/dynamic_cp_scheduler.py:112-286``
        and its use in the Megatron engine). All ranks of the CP group hold the same batch; the scheduler packs its samples
        into micro-batches in which each sample is owned by an aligned sub-group of 1, 2, 4, ... ranks. A rank runs only the
        samples of its sub-group; the leaders' outputs are summed back over the CP group so that every rank returns the
        whole batch, as with the static layout. A sub-group of width k sees each of its gradients k-fold (the output gather
        scales by k) and its samples are seen by k of the ``cp`` ranks only, so the loss is scaled by cp / k: after the
        data-parallel average every sample then counts once, exactly as in the static layout."""
        from verl_b200.utils.dynamic_cp_scheduler import DynamicCPScheduler

        batch = data.batch
        meta = dict(getattr(data, "meta_info", {}) or {})
        dev = self.device
        tensors = {k: (_to_device(v, dev) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        n = tensors["input_ids"].shape[0]
        seq_lens = tensors["attention_mask"].sum(-1)
        lens = [max(1, int(x)) for x in seq_lens.tolist()]
        cp = self.sp_size
        cap = int(cfg_get(self.engine_config, "max_seqlen_per_dp_cp_rank", 0) or 0)
        if cap <= 0:
            cap = int(meta.get("max_token_len_per_gpu", 0) or 0) or -(-max(lens) // cp)
        cap = max(cap, -(-max(lens) // cp))                  # the longest sample must fit the full group
        plan = DynamicCPScheduler(cap, 1, cp).schedule(lens, self.sp_rank, cp_layout="zigzag" if self._cp_zigzag else "contiguous")
        info: dict[str, Any] = {"dp_size": self.dp_size}
        if not forward_only and loss_function is not None:
            mask_key = "response_mask" if "response_mask" in tensors else None
            ntok = tensors[mask_key].sum().to(torch.float32) if mask_key else seq_lens.sum().to(torch.float32)
            cnt = torch.stack([ntok, torch.tensor(float(n), device=dev)])
            dist.all_reduce(cnt, group=self.dp_group)
            info["batch_num_tokens"], info["global_batch_size"] = cnt[0], cnt[1]
            self._alloc_grads()
        full: dict[str, torch.Tensor] = {}
        metrics: dict[str, Metric] = {}
        losses = []
        self.model.train(not forward_only)
        self.dcp_stats = {"micro_batches": len(plan), "group_sizes": [mb["local_cp_size"] for mb in plan if mb["sample_ids"]]}
        for mbp in plan:
            idxs = mbp["sample_ids"]
            if not idxs:
                continue
            k = mbp["local_cp_size"]
            it = torch.as_tensor(idxs, device=dev)
            mb = {key: (v.index_select(0, it) if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == n else v) for key, v in tensors.items()}
            with (torch.no_grad() if forward_only else torch.enable_grad()), self._sub_sp(k, mbp["cp_rank"]):
                mo = self._forward_micro_batch(mb, meta)
                if loss_function is not None:
                    mb_data = dict(mb)
                    mb_data.update(info)
                    loss, m = loss_function(model_output=mo, data=mb_data, dp_group=self.dp_group)
                    if not forward_only:
                        (loss * (cp / k)).backward()
                    if mbp["group_leader"]:
                        losses.append(float(loss.detach()))
                        for key, v in m.items():
                            if key in metrics:
                                metrics[key].append(v)
                            else:
                                metrics[key] = v if isinstance(v, Metric) else Metric(AggregationType.MEAN, v)
            if mbp["group_leader"]:
                for key, v in mo.items():
                    if key not in full:
                        full[key] = torch.zeros(n, *v.shape[1:], dtype=v.dtype, device=v.device)
                    full[key].index_copy_(0, it, v.detach())
        if not forward_only and loss_function is not None:
            self.store.fold_autograd_grads()
        # every rank of the CP group returns the whole batch: exchange what the leaders hold (host side first: which outputs exist)
        mine = {"keys": {key: (tuple(v.shape[1:]), str(v.dtype).split(".")[-1]) for key, v in full.items()}, "loss": losses,
                "metrics": {key: (v.aggregation.value, list(v.values)) for key, v in metrics.items()}}
        everyone = [None] * cp
        dist.all_gather_object(everyone, mine, group=self._sp_host_group())
        keys = {}
        for e in everyone:
            keys.update(e["keys"])
        model_output = {}
        for key in sorted(keys):
            shape, dt = keys[key]
            t = full.get(key)
            if t is None:
                t = torch.zeros(n, *shape, dtype=getattr(torch, dt), device=dev)
            dist.all_reduce(t, group=self._dcp_groups[cp])
            model_output[key] = t
        losses = [x for e in everyone for x in e["loss"]]
        merged: dict[str, Metric] = {}
        for e in everyone:
            for key, (agg, vals) in e["metrics"].items():
                merged.setdefault(key, Metric(agg)).append(list(vals))
        return {"model_output": model_output, "loss": losses, "metrics": merged}

    def _alloc_grads(self):
        s = self.store
        if self._symm_grads is not None and s.grad is None:
            s.grad = self._symm_grads.tensor(torch.float32, s.total)
            for p, o in zip(s.params, s.offsets):
                p.main_grad = s.grad[o : o + p.numel()].view(p.shape)
        else:
            s.alloc_grads()

    def optimizer_zero_grad(self):
        self._alloc_grads()
        self.store.zero_grads()

    # ------------------------------------------------------------------ optimizer step
    @torch.no_grad()
    def optimizer_step(self) -> float:
        s = self.store
        assert s.grad is not None, "optimizer_step without gradients"
        W = self.fsdp_size
        if self._symm_grads is not None:
            return self._optimizer_step_fused()
        # 1. reduce gradients: average over data-parallel ranks, keep only this rank's shard
        if W > 1 or self.ddp_group is not None:
            if s.grad.is_cuda:
                if W > 1:
                    if self.grad_shard is None:
                        self.grad_shard = torch.empty(s.shard_size, dtype=torch.float32, device=self.device)
                    dist.reduce_scatter_tensor(self.grad_shard, s.grad, op=dist.ReduceOp.AVG, group=self.fsdp_group)
                    gshard = self.grad_shard
                else:
                    gshard = s.grad
                if self.ddp_group is not None:
                    dist.all_reduce(gshard, op=dist.ReduceOp.AVG, group=self.ddp_group)
            else:
                if W > 1:
                    dist.all_reduce(s.grad, group=self.fsdp_group)
                if self.ddp_group is not None:
                    dist.all_reduce(s.grad, group=self.ddp_group)
                s.grad.div_(W * self.ddp_size)
                gshard = s.grad[s.shard_slice]
        else:
            gshard = s.grad
        # 2. global gradient norm
        native = gshard.is_cuda and _ext.available()
        if native:
            self._sumsq.zero_()
            _ext.ops().sqnorm_(gshard, self._sumsq)
            sumsq = self._sumsq
        else:
            sumsq = gshard.float().pow(2).sum().reshape(1)
        if W > 1:
            dist.all_reduce(sumsq, group=self.fsdp_group)
        sumsq = self._sumsq_across_model_parallel(sumsq, gshard)
        grad_norm = self._adamw_update(gshard, sumsq, native)
        # 3. all-gather the updated working copy
        if W > 1:
            if s.flat.is_cuda:
                dist.all_gather_into_tensor(s.flat, s.flat[s.shard_slice].clone(), group=self.fsdp_group)
            else:
                parts = [torch.empty(s.shard_size, dtype=s.flat.dtype) for _ in range(W)]
                dist.all_gather(parts, s.flat[s.shard_slice].clone(), group=self.fsdp_group)
                s.flat.copy_(torch.cat(parts))
        s.zero_grads()
        return grad_norm

    def _adamw_update(self, gshard: torch.Tensor, sumsq: torch.Tensor, native: bool) -> float:
        """Clip by the global norm ``sqrt(sumsq)`` and apply AdamW to this rank's slice (fp32 master → working copy)."""
        s = self.store
        self.step_count += 1
        lr = self.current_lr()
        if native:
            _ext.ops().clip_coef_(sumsq, self.clip_grad, self._scalars)
            _ext.ops().adamw_(self.master, self.exp_avg, self.exp_avg_sq, gshard, s.flat[s.shard_slice] if s.flat.dtype == torch.bfloat16 else None,
                              lr, self.beta1, self.beta2, self.adam_eps, self.weight_decay, self.step_count, self._scalars)
            if s.flat.dtype != torch.bfloat16:
                s.flat[s.shard_slice].copy_(self.master)
            sc = self._scalars.tolist()
            grad_norm, skipped = sc[2], sc[1] != 0.0
        else:
            grad_norm = float(sumsq.sqrt())
            skipped = not math.isfinite(grad_norm)
            if not skipped:
                coef = min(1.0, self.clip_grad / (grad_norm + 1e-6)) if self.clip_grad > 0 else 1.0
                _adamw_reference(self.master, self.exp_avg, self.exp_avg_sq, gshard, lr, self.beta1, self.beta2,
                                 self.adam_eps, self.weight_decay, self.step_count, coef)
                s.flat[s.shard_slice].copy_(self.master.to(s.flat.dtype))
        if skipped:
            self.step_count -= 1
            print(f"WARN: rank {self.rank} grad_norm is not finite: {grad_norm}; skipping optimizer step")
        return grad_norm

    def _sumsq_across_model_parallel(self, sumsq: torch.Tensor, gshard: torch.Tensor) -> torch.Tensor:
        """Hook for engines whose parameters are also split over tensor/pipeline ranks; a no-op for pure data parallelism."""
        return sumsq

    @torch.no_grad()
    def _optimizer_step_fused(self) -> float:
        """Reduce-scatter (+1/W, +Σg²) by peer loads → scalar all-reduce → AdamW whose epilogue stores the new bf16
        values into every rank's parameter buffer (the all-gather). Three kernels and two device barriers in total."""
        s, o = self.store, _ext.ops()
        W, off = self.world, self.rank * s.shard_size
        if self.grad_shard is None:
            self.grad_shard = torch.empty(s.shard_size, dtype=torch.float32, device=self.device)
        self._symm_grads.barrier()                       # every rank has finished writing its gradients
        self._sumsq.zero_()
        o.symm_reduce_scatter(self._symm_grads.table(), W, off, self.grad_shard, self._sumsq, 1.0 / W)
        dist.all_reduce(self._sumsq, group=self.fsdp_group)
        self.step_count += 1
        lr = self.current_lr()
        o.clip_coef_(self._sumsq, self.clip_grad, self._scalars)
        o.symm_adamw_allgather(self.master, self.exp_avg, self.exp_avg_sq, self.grad_shard, self._symm_params.table(), W, off, lr,
                               self.beta1, self.beta2, self.adam_eps, self.weight_decay, self.step_count, self._scalars)
        self._symm_params.barrier()                      # all shards of the new parameters have landed everywhere
        sc = self._scalars.tolist()
        if sc[1] != 0.0:
            self.step_count -= 1
            print(f"WARN: rank {self.rank} grad_norm is not finite: {sc[2]}; skipping optimizer step")
        s.zero_grads()
        return sc[2]

    def lr_scheduler_step(self) -> float:
        self.sched_step += 1
        return self.current_lr()

    # ------------------------------------------------------------------ weights out
    def get_per_tensor_param(self, **kwargs):
        """(HF name, full tensor) pairs. Parameters are resident in full on every rank, so this is a view walk —
        no collective (the reference all-gathers every DTensor here: fsdp/transformer_impl.py:1033-1039)."""
        if not self.store.flat.is_cuda and self.device.type == "cuda":
            self.to("cuda", model=True, optimizer=False, grad=False)
        if getattr(self.model, "lora_config", None):
            from verl_b200.models.lora import merged_hf_named_tensors

            return merged_hf_named_tensors(self.model), None
        return self.model.hf_named_tensors(), None

    # ------------------------------------------------------------------ checkpoint
    def export_weights_source(self, file_path: Optional[str] = None) -> dict:
        """Description of the current bf16 weights that a rollout replica in ANOTHER process can pull
        (``AsyncRolloutServer.update_weights``). On CUDA the flat parameter buffer is copied into an export buffer that was
        allocated outside the caching allocator and its CUDA IPC handle is returned: the replica maps it and copies
        device-to-device over NVLink, no collective spans the two jobs. On CPU (or with ``file_path`` given) the buffer is
        written to a file instead."""
        s = self.store
        layout = {"names": list(s.names), "shapes": [list(p.shape) for p in s.params], "offsets": [int(o) for o in s.offsets],
                  "dtype": str(s.flat.dtype).replace("torch.", "")}
        if s.flat.is_cuda and file_path is None:
            import base64

            from verl_b200.ops import _ext

            ops_ = _ext.ops()
            nbytes = s.flat.numel() * s.flat.element_size()
            if getattr(self, "_export_ptr", None) is None:
                self._export_ptr = int(ops_.symm_alloc(nbytes))
                self._export_handle = base64.b64encode(ops_.ipc_get_handle(self._export_ptr).numpy().tobytes()).decode()
            ops_.tensor_from_ptr(self._export_ptr, [s.flat.numel()], s.flat.dtype).copy_(s.flat)
            torch.cuda.synchronize()
            return {"kind": "cuda_ipc", "handle": self._export_handle, "nbytes": nbytes, **layout}
        assert file_path is not None, "a file path is needed to export weights from a CPU engine"
        tmp = file_path + ".tmp"
        torch.save({"flat": s.flat.detach().to("cpu"), **layout}, tmp)
        os.replace(tmp, file_path)
        return {"kind": "file", "path": file_path}

    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None, **kwargs):
        self.checkpoint_manager.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False, **kwargs):
        self._host_flat = None           # a cached pinned copy of frozen weights would be stale after this
        self.checkpoint_manager.load_checkpoint(local_path, hdfs_path, del_local_after_load)


@EngineRegistry.register(model_type="value_model", backend=["fsdp", "fsdp2"], device=["cuda", "cpu"])
class FSDPEngineWithValueHead(FSDPEngine):
    """Same trunk with a scalar head (critic / reward model): outputs ``values`` instead of log-probs."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._value_head = True
