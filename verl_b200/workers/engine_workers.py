"""Role workers that sit between the trainer and the engines.

* :class:`TrainingWorker` — one trainable or frozen model behind the engine contract (mini-batch loop, metrics).
* :class:`ActorRolloutRefWorker` — the colocated "hybrid engine": actor + reference policy + in-house rollout engine in
  one process per GPU, sharing the resident bf16 weights between training and generation.

Parity target: ``verl/workers/engine_workers.py`` (TrainingWorker :160-450, ActorRolloutRefWorker :453-848).
"""

from __future__ import annotations

import os
import time
from functools import partial
from typing import Any, Optional

import numpy as np
import torch
import torch.distributed as dist

from verl_b200.protocol import DataProto, TensorBatch
from verl_b200.single_controller.base import Dispatch, Worker, register
from verl_b200.single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn
from verl_b200.utils.device import get_device_name
from verl_b200.utils.flops_counter import FlopsCounter
from verl_b200.utils.metric import AggregationType, Metric
from verl_b200.utils.torch_functional import compute_position_id_with_mask
from verl_b200.workers.engine.base import EngineRegistry
from verl_b200.workers.engine.fsdp.engine import IO_STATS, cfg_get
from verl_b200.workers.utils.losses import ppo_loss, value_loss

__all__ = ["TrainingWorker", "ActorRolloutRefWorker", "CriticWorker", "ensure_process_group"]


def ensure_process_group(timeout_s: int = 600):
    """Join the global process group described by the launcher's environment (no-op for world size 1)."""
    import datetime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if torch.cuda.is_available():
            lr = int(os.environ.get("LOCAL_RANK", "0")) % torch.cuda.device_count()
            torch.cuda.set_device(lr)
            dist.init_process_group("cpu:gloo,cuda:nccl", timeout=datetime.timedelta(seconds=timeout_s))
        else:
            dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=timeout_s))


def _model_inputs(data) -> dict:
    """Non-tensor columns that the engines consume: the per-row image inputs of vision-language models."""
    nt = getattr(data, "non_tensor_batch", None) or {}
    return {"multi_modal_inputs": nt["multi_modal_inputs"]} if "multi_modal_inputs" in nt else {}


class TrainingWorker(Worker):
    """Mini-batch / epoch loop around one engine. ``config`` keys: model_type, backend, model, engine, optim, checkpoint
    plus the batching knobs (ppo_mini_batch_size, ppo_epochs, micro-batch / dynamic-bsz settings)."""

    def __init__(self, config, role: str = "actor"):
        super().__init__()
        ensure_process_group(int(cfg_get(config, "nccl_timeout", 600)))
        self.config = config
        self.role = role
        self.engine = EngineRegistry.new(cfg_get(config, "model_type", "language_model"), cfg_get(config, "backend", "fsdp"),
                                         model_config=cfg_get(config, "model"), engine_config=cfg_get(config, "engine"),
                                         optimizer_config=cfg_get(config, "optim"), checkpoint_config=cfg_get(config, "checkpoint"))
        self.loss_fn = None
        self.flops_counter: Optional[FlopsCounter] = None
        self._mesh_registered = False

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def reset(self):
        self.engine.initialize()
        self.flops_counter = FlopsCounter(self.engine.cfg)
        if not self._mesh_registered:
            self._register_dispatch_collect_info(self.role, dp_rank=self.engine.get_data_parallel_rank(),
                                                 is_collect=self.engine.is_mp_src_rank_with_outputs())
            self._mesh_registered = True

    def set_loss_fn(self, loss_fn):
        self.loss_fn = loss_fn

    # ------------------------------------------------------------------ helpers
    def _batch_meta(self, data: DataProto, prefix: str) -> dict:
        """Micro-batching + sampling knobs for the engine, resolved from the worker config and the call's meta_info."""
        c = self.config
        meta = dict(data.meta_info)
        if "use_dynamic_bsz" not in meta:
            meta["use_dynamic_bsz"] = bool(cfg_get(c, f"{prefix}use_dynamic_bsz", cfg_get(c, "use_dynamic_bsz", False)))
        if meta["use_dynamic_bsz"]:
            meta.setdefault("max_token_len_per_gpu", int(cfg_get(c, f"{prefix}max_token_len_per_gpu", cfg_get(c, "ppo_max_token_len_per_gpu", 16384))))
        else:
            mbs = cfg_get(c, f"{prefix}micro_batch_size_per_gpu", cfg_get(c, "ppo_micro_batch_size_per_gpu", None))
            meta.setdefault("micro_batch_size_per_gpu", int(mbs) if mbs else len(data))
        meta.setdefault("use_prefix_grouper", bool(cfg_get(c, "use_prefix_grouper", False)))
        if prefix != "ppo_":
            meta.pop("score_centering", None)      # only the update pass computes the centering term
        return meta

    def _postprocess_metrics(self, metrics: dict, n_tokens: int, dt: float, forward_only: bool) -> dict:
        out = {k: (v.aggregate() if isinstance(v, Metric) else v) for k, v in metrics.items()}
        if self.flops_counter is not None and dt > 0:
            est, promised = self.flops_counter.estimate_flops([n_tokens], dt)
            out[f"perf/mfu/{self.role}"] = est / promised / (3.0 if forward_only else 1.0)
        if torch.cuda.is_available():
            out[f"perf/max_memory_allocated_gb/{self.role}"] = torch.cuda.max_memory_allocated() / 1024**3
        return out

    # ------------------------------------------------------------------ compute
    def train_mini_batch(self, data: DataProto) -> dict:
        """Split the local batch into mini-batches (one optimizer step each), repeated ``ppo_epochs`` times."""
        c = self.config
        eng = self.engine
        dp = eng.get_data_parallel_size()
        n_local = len(data)
        mini_global = int(cfg_get(c, "ppo_mini_batch_size", n_local * dp))
        mini = max(1, min(n_local, mini_global // dp))
        epochs = int(cfg_get(c, "ppo_epochs", 1))
        shuffle = bool(cfg_get(c, "shuffle", False))
        meta = self._batch_meta(data, "ppo_")
        all_metrics: dict[str, Metric] = {}
        t0 = time.perf_counter()
        with eng.train_mode():
            n_steps = epochs * ((n_local + mini - 1) // mini)
            step_i = 0
            for ep in range(epochs):
                order = torch.randperm(n_local, generator=torch.Generator().manual_seed(int(cfg_get(c, "data_loader_seed", 42)) + ep + eng.get_data_parallel_rank())) \
                    if shuffle else torch.arange(n_local)
                for s in range(0, n_local, mini):
                    mb = data.select_idxs(order[s : s + mini])
                    mb.meta_info = meta
                    out = eng.train_batch(mb, self.loss_fn)
                    step_i += 1
                    for k, v in out["metrics"].items():
                        if k == "grad_norm":
                            k, v = f"{self.role}/grad_norm", Metric(AggregationType.MEAN, v)
                        if k in all_metrics:
                            all_metrics[k].append(v)
                        else:
                            all_metrics[k] = v if isinstance(v, Metric) else Metric(AggregationType.MEAN, v)
                    if step_i == n_steps:
                        all_metrics[f"{self.role}/lr"] = Metric(AggregationType.MEAN, eng.lr_scheduler_step())
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if getattr(eng, "_symm_grads", None) is None:
            eng.store.free_grads()   # the fp32 gradient buffer is only needed inside an update; the KV cache wants the room
        dt = time.perf_counter() - t0
        n_tok = int(data.batch["attention_mask"].sum()) * epochs
        return self._postprocess_metrics(all_metrics, n_tok, dt, forward_only=False)

    def infer_batch(self, data: DataProto, prefix: str = "log_prob_") -> dict:
        meta = self._batch_meta(data, prefix)
        data = DataProto(batch=data.batch, non_tensor_batch=data.non_tensor_batch, meta_info=meta)
        with self.engine.eval_mode():
            return self.engine.infer_batch(data, None)

    # ------------------------------------------------------------------ placement / checkpoint
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def to(self, device, model=True, optimizer=True, grad=True):
        self.engine.to(device, model=model, optimizer=optimizer, grad=grad)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        self.engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False):
        self.engine.load_checkpoint(local_path, hdfs_path, del_local_after_load)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def wait_checkpoint(self):
        _wait_checkpoint(self.engine)


def _wait_checkpoint(engine):
    """Join this rank's background checkpoint writer (asynchronous saves), then meet the other ranks."""
    mgr = getattr(engine, "checkpoint_manager", None)
    if mgr is not None and hasattr(mgr, "wait_async_save"):
        mgr.wait_async_save()
    if dist.is_initialized():
        dist.barrier()


def _to_host(t: torch.Tensor) -> torch.Tensor:
    if t.is_cuda:
        IO_STATS["d2h_bytes"] += t.numel() * t.element_size()
    return t.cpu()


def _mini_batch_trajectories(mini_prompts, n):
    """``ppo_mini_batch_size`` counts PROMPTS (it is compared with ``data.train_batch_size``); every prompt contributes
    ``rollout.n`` trajectories, so one optimizer step covers ``mini * n`` rows of the rollout batch (reference:
    ``verl/trainer/ppo/ray_trainer.py:1352-1363`` for the actor, ``:1382`` for the critic). None stays None (= one step)."""
    if mini_prompts is None:
        return None
    return int(mini_prompts) * max(1, int(n or 1))


def _role_cfg(full, role: str, model_type: str):
    """Flatten the reference-style config tree (actor_rollout_ref.{model,actor,ref,rollout} / critic) into the keys a
    TrainingWorker reads."""
    if role == "critic":
        c = full
        strategy = cfg_get(c, "strategy", "fsdp")
        eng = dict(cfg_get(c, "fsdp_config", {}) or {}) if strategy.startswith("fsdp") else dict(cfg_get(c, "megatron", {}) or {})
        return {"model_type": "value_model", "backend": strategy, "model": cfg_get(c, "model"), "engine": eng, "optim": cfg_get(c, "optim"),
                "checkpoint": cfg_get(c, "checkpoint"), "ppo_mini_batch_size": _mini_batch_trajectories(cfg_get(c, "ppo_mini_batch_size"), cfg_get(c, "rollout_n", 1)),
                "ppo_epochs": cfg_get(c, "ppo_epochs", 1), "shuffle": cfg_get(c, "shuffle", False),
                "use_dynamic_bsz": cfg_get(c, "use_dynamic_bsz", False), "ppo_max_token_len_per_gpu": cfg_get(c, "ppo_max_token_len_per_gpu"),
                "ppo_micro_batch_size_per_gpu": cfg_get(c, "ppo_micro_batch_size_per_gpu"),
                "log_prob_micro_batch_size_per_gpu": cfg_get(c, "forward_micro_batch_size_per_gpu", cfg_get(c, "ppo_micro_batch_size_per_gpu")),
                "log_prob_max_token_len_per_gpu": cfg_get(c, "forward_max_token_len_per_gpu"), "nccl_timeout": cfg_get(c, "nccl_timeout", 600)}
    sub = cfg_get(full, role)
    strategy = cfg_get(sub, "strategy", "fsdp")
    eng = dict(cfg_get(sub, "fsdp_config", {}) or {}) if strategy.startswith("fsdp") else dict(cfg_get(sub, "megatron", {}) or {})
    out = {"model_type": model_type, "backend": strategy, "model": cfg_get(full, "model"), "engine": eng,
           "checkpoint": cfg_get(sub, "checkpoint"), "nccl_timeout": cfg_get(full, "nccl_timeout", 600),
           # one switch for actor update, old log-probs and reference log-probs (reference: actor.use_prefix_grouper)
           "use_prefix_grouper": bool(cfg_get(cfg_get(full, "actor"), "use_prefix_grouper", False))}
    if role == "actor":
        out.update({k: cfg_get(sub, k) for k in ("ppo_mini_batch_size", "ppo_epochs", "shuffle", "use_dynamic_bsz", "data_loader_seed",
                                                 "ppo_max_token_len_per_gpu", "ppo_micro_batch_size_per_gpu")})
        out["optim"] = cfg_get(sub, "optim")
        ro = cfg_get(full, "rollout")
        out["ppo_mini_batch_size"] = _mini_batch_trajectories(out["ppo_mini_batch_size"], cfg_get(ro, "n", 1))
        out["log_prob_micro_batch_size_per_gpu"] = cfg_get(ro, "log_prob_micro_batch_size_per_gpu", cfg_get(sub, "ppo_micro_batch_size_per_gpu"))
        out["log_prob_use_dynamic_bsz"] = cfg_get(ro, "log_prob_use_dynamic_bsz", cfg_get(sub, "use_dynamic_bsz", False))
        out["log_prob_max_token_len_per_gpu"] = cfg_get(ro, "log_prob_max_token_len_per_gpu", cfg_get(sub, "ppo_max_token_len_per_gpu"))
    else:  # ref: frozen
        eng["forward_only"] = True
        out["optim"] = None
        for k in ("log_prob_micro_batch_size_per_gpu", "log_prob_use_dynamic_bsz", "log_prob_max_token_len_per_gpu"):
            out[k] = cfg_get(sub, k)
    return out


def _annotate(message: str, role: str):
    from verl_b200.utils.profiler import DistProfiler

    return DistProfiler.annotate(message=message, role=role)


def _role_profiler(config, *roles):
    """``DistProfiler`` of a role worker: the union of the ``profiler`` sections of the roles this process plays (reference:
    ``verl/workers/engine_workers.py:262-290`` merges actor / rollout / ref profiler configs the same way)."""
    from verl_b200.utils.profiler import DistProfiler, ProfilerConfig

    known = set(ProfilerConfig.__dataclass_fields__)
    merged = None
    for r in roles:
        sec = cfg_get(config, f"{r}.profiler", None) if r else cfg_get(config, "profiler", None)
        if sec is None:
            continue
        d = {k: (sec.get(k) if hasattr(sec, "get") else getattr(sec, k, None)) for k in known}
        d = {k: v for k, v in d.items() if v is not None}
        tool = d.get("tool")
        tc = d.get("tool_config")
        if tool and tc is not None and hasattr(tc, "get") and tc.get(tool) is not None:
            d["tool_config"] = dict(tc.get(tool))         # the per-tool subsection of the role's tool_config
        elif tc is not None and hasattr(tc, "keys"):
            d["tool_config"] = dict(tc)
        d["ranks"] = list(d.get("ranks") or [])
        pc = ProfilerConfig(**d)
        merged = pc if merged is None else merged.union(pc)
    return DistProfiler(int(os.environ.get("RANK", "0")), merged)


class _ProfiledWorker:
    """``start_profile`` / ``stop_profile`` group calls of a role worker (the trainer brackets the steps listed in
    ``global_profiler.steps`` with them)."""

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def start_profile(self, **kwargs) -> None:
        self.profiler.start(**kwargs)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def stop_profile(self) -> None:
        self.profiler.stop()


class ActorRolloutRefWorker(Worker, _ProfiledWorker):
    """Colocated actor / reference / rollout roles of one GPU. ``role`` ∈ {actor, ref, rollout, actor_rollout,
    actor_rollout_ref}; ``config`` is the ``actor_rollout_ref`` subtree."""

    actor_worker_cls = TrainingWorker      # subclasses may substitute a worker with more primitives (engine_workers_tinker)

    def __init__(self, config, role: str = "actor_rollout_ref"):
        super().__init__()
        ensure_process_group(int(cfg_get(config, "nccl_timeout", 600)))
        self.config = config
        self.role = role
        self._is_actor = "actor" in role
        self._is_rollout = "rollout" in role
        self._is_ref = "ref" in role
        self.actor: Optional[TrainingWorker] = None
        self.ref: Optional[TrainingWorker] = None
        self.rollout = None
        self.device = torch.device(get_device_name())
        self.profiler = _role_profiler(config, *[r for r, on in (("actor", self._is_actor), ("rollout", self._is_rollout), ("ref", self._is_ref)) if on])

    # ------------------------------------------------------------------ build
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        c = self.config
        if self._is_ref:
            self.ref = TrainingWorker(_role_cfg(c, "ref", "language_model"), role="ref")
            self.ref.reset()
        dcfg = cfg_get(c, "distillation", None)
        self.teacher = None
        # teacher_mode=server: the teachers run on rollout servers of their own and the trainer fetches their top-k heads itself
        self._distill = bool(dcfg is not None and cfg_get(dcfg, "enable", False) and self._is_actor)
        if self._distill and str(cfg_get(dcfg, "teacher_mode", "colocated")) == "colocated":
            # frozen teacher colocated with the student (same engine type as the reference policy, its own weights)
            tcfg = _role_cfg(c, "ref" if cfg_get(c, "ref", None) is not None else "actor", "language_model")
            tcfg = dict(tcfg, model=cfg_get(dcfg, "teacher_model"), optim=None)
            tcfg["engine"] = dict(tcfg.get("engine") or {}, forward_only=True)
            self.teacher = TrainingWorker(tcfg, role="teacher")
            self.teacher.reset()
        if self._is_actor:
            self.actor = self.actor_worker_cls(_role_cfg(c, "actor", "language_model"), role="actor")
            self.actor.reset()
            self.actor.set_loss_fn(partial(ppo_loss, cfg_get(c, "actor"), distillation=dcfg))
            eng = self.actor.engine
            self._register_dispatch_collect_info("actor", dp_rank=eng.get_data_parallel_rank(), is_collect=eng.is_mp_src_rank_with_outputs())
        if self._is_ref and not self._is_actor:
            eng = self.ref.engine
            self._register_dispatch_collect_info("actor", dp_rank=eng.get_data_parallel_rank(), is_collect=eng.is_mp_src_rank_with_outputs())
        if self._is_rollout:
            self._build_rollout()
        tp = getattr(self, "_rollout_tp", 1) if self._is_rollout else 1
        self._register_dispatch_collect_info("rollout", dp_rank=self.rank // tp, is_collect=self.rank % tp == 0)

    def _build_rollout(self):
        from verl_b200.workers.rollout.engine import InferenceEngine

        ro = cfg_get(self.config, "rollout")
        src = self.actor if self.actor is not None else self.ref
        model = src.engine.model
        self._rollout_owns_model = False
        lora_needs_merge = bool(getattr(model, "lora_config", None)) and (int(cfg_get(ro, "tensor_model_parallel_size", 1) or 1) > 1 or cfg_get(ro, "quantization", None))
        if getattr(src.engine, "tp_size", 1) * getattr(src.engine, "pp_size", 1) > 1 or getattr(src.engine, "_zero3_rows", None) or lora_needs_merge:
            # the trainer holds only a tensor/pipeline shard (or ZeRO-3 row shards), or low-rank adapters that a tensor-parallel / fp8
            # replica cannot apply unmerged: the rollout replica keeps its own full copy, refreshed by update_weights() from the engine's
            # per-tensor export (which folds adapters in). A bf16 replica without tensor parallelism serves adapters unmerged instead.
            from verl_b200.models.transformer import DecoderLM

            if src.engine.cfg.vision:
                from verl_b200.models.vision import VisionLanguageModel

                model = VisionLanguageModel(src.engine.cfg, dtype=src.engine.dtype, device=src.engine.device, init=False)
            else:
                model = DecoderLM(src.engine.cfg, dtype=src.engine.dtype, device=src.engine.device, init=False)
            model.load_hf_stream(src.engine.get_per_tensor_param()[0])
            self._rollout_owns_model = True
        max_len = cfg_get(ro, "max_model_len", None) or (int(cfg_get(ro, "prompt_length", 512)) + int(cfg_get(ro, "response_length", 512)))
        self._rollout_tp = int(cfg_get(ro, "tensor_model_parallel_size", 1) or 1)
        tp_group = tp_ctx = None
        if self._rollout_tp > 1:
            model, tp_group, tp_ctx = self._build_rollout_tp(model, ro)
        self.rollout = InferenceEngine(
            model, max_num_seqs=int(cfg_get(ro, "max_num_seqs", 256)), max_model_len=int(max_len),
            max_num_batched_tokens=int(cfg_get(ro, "max_num_batched_tokens", 8192)),
            gpu_memory_utilization=float(cfg_get(ro, "gpu_memory_utilization", 0.5)), enforce_eager=bool(cfg_get(ro, "enforce_eager", False)),
            sync_interval=int(cfg_get(ro, "sync_interval", 16)), enable_prefix_sharing=bool(cfg_get(ro, "enable_prefix_caching", True)),
            num_blocks=cfg_get(ro, "num_blocks", None), tp_group=tp_group, tp_ctx=tp_ctx, quantization=cfg_get(ro, "quantization", None),
            enable_chunked_prefill=bool(cfg_get(ro, "enable_chunked_prefill", True)),
            enable_prefix_caching=bool(cfg_get(ro, "enable_prefix_caching", True)))

    def _build_rollout_tp(self, full_model, ro):
        """Rollout replicas of ``tp`` adjacent ranks: every rank keeps a tensor-parallel slice of the decoder layers cut from
        the full weights it holds for training (reference: vLLM ``tensor_parallel_size`` replicas,
        ``verl/workers/rollout/replica.py:102-106``)."""
        from verl_b200.models.parallel_model import build_rollout_shard
        from verl_b200.parallel.tp import TPContext, fused_comm_enabled

        tp, world, rank = self._rollout_tp, dist.get_world_size(), dist.get_rank()
        assert world % tp == 0, "world size must be a multiple of rollout.tensor_model_parallel_size"
        mine = host = None
        cuda = torch.cuda.is_available()
        for b in range(0, world, tp):
            ranks = list(range(b, b + tp))
            g = dist.new_group(ranks)
            hgrp = dist.new_group(ranks, backend="gloo") if cuda else g
            if rank in ranks:
                mine, host = g, hgrp
        if hasattr(full_model, "visual") and hasattr(full_model, "language_model"):
            # vision-language model: the decoder is cut, the tower stays whole on every rank of the replica
            from verl_b200.models.parallel_model import VisionLanguageRolloutShard

            local = VisionLanguageRolloutShard(full_model, rank % tp, tp)
            self._rollout_sync_target = full_model          # a replica-owned copy is refreshed as a whole (tower included) ...
            full_model = full_model.language_model          # ... and update_weights() re-cuts the decoder slice from its decoder
        else:
            local = build_rollout_shard(full_model, rank % tp, tp)
        self._rollout_full_model = full_model
        ctx = None
        if cuda and fused_comm_enabled():
            max_tok = int(cfg_get(ro, "max_num_batched_tokens", 8192))
            ctx = TPContext(mine, host, max_tokens=max(max_tok, int(cfg_get(ro, "max_num_seqs", 256))), hidden=full_model.cfg.hidden_size,
                            max_out=full_model.cfg.hidden_size, graph_safe=True)
        return local, mine, ctx

    # ------------------------------------------------------------------ rollout
    def _agent_loop_manager(self):
        """Server-mode rollout inside this worker: the engine is wrapped in a hybrid replica and the agent loops of this
        rank's share of the batch run against it (the reference reaches its servers through Ray actors instead:
        verl/experimental/agent_loop/agent_loop.py:1190-1312)."""
        if getattr(self, "_agent_mgr", None) is None:
            from verl_b200.experimental.agent_loop import AgentLoopManager
            from verl_b200.utils.tokenizer import ByteChatTokenizer, hf_tokenizer
            from verl_b200.workers.rollout.llm_server import LLMServerManager
            from verl_b200.workers.rollout.replica import RolloutReplica

            path = cfg_get(self.config, "model.path", None)
            if path and os.path.isdir(os.path.expanduser(path)):
                tok = hf_tokenizer(os.path.expanduser(path))
            else:
                tok = ByteChatTokenizer()
            eos = getattr(tok, "eos_token_id", None)
            fully_async = str(cfg_get(self.config, "rollout.agent.client", "sync")) == "fully_async"
            self._replica = RolloutReplica(self.rank, cfg_get(self.config, "rollout")).init_hybrid(self.rollout, eos_token_id=eos, tokenizer=tok)
            self._agent_mgr = AgentLoopManager(self.config, LLMServerManager([self._replica], fully_async=fully_async), tok)
        return self._agent_mgr

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("rollout"))
    @_annotate("generate_sequences", "rollout")
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        """Left-padded prompts in → prompts + right-padded responses out (with rollout log-probs)."""
        from verl_b200.workers.rollout.engine import SamplingParams

        ro = cfg_get(self.config, "rollout")
        if str(cfg_get(ro, "mode", "sync")) == "async" or bool(cfg_get(ro, "multi_turn.enable", False)):
            return self._agent_loop_manager().generate_sequences(prompts)
        meta = prompts.meta_info
        ids = prompts.batch["input_ids"]
        att = prompts.batch["attention_mask"]
        bs, P = ids.shape
        R = int(meta.get("response_length", cfg_get(ro, "response_length", 512)))
        do_sample = meta.get("do_sample", cfg_get(ro, "do_sample", True))
        validate = meta.get("validate", False)
        vk = cfg_get(ro, "val_kwargs", {}) or {}
        temperature = float(cfg_get(vk, "temperature", 0.0)) if validate else float(meta.get("temperature", cfg_get(ro, "temperature", 1.0)))
        sp = SamplingParams(
            temperature=temperature if do_sample or validate else 0.0,
            top_p=float(cfg_get(vk, "top_p", 1.0)) if validate else float(meta.get("top_p", cfg_get(ro, "top_p", 1.0))),
            top_k=int(cfg_get(vk, "top_k", -1)) if validate else int(meta.get("top_k", cfg_get(ro, "top_k", -1))),
            max_tokens=R, ignore_eos=bool(cfg_get(ro, "ignore_eos", False)), top_logprobs=0 if validate else int(cfg_get(ro, "topk_log_probs", 0) or 0), seed=int(meta.get("seed", 0)) + 1000003 * (self.rank // getattr(self, "_rollout_tp", 1)) + int(meta.get("global_steps", 0)))
        eos = meta.get("eos_token_id", None)
        pad_id = int(meta.get("pad_token_id", 0) or 0)
        ids_cpu, att_cpu = ids.cpu(), att.cpu().bool()
        plist = [ids_cpu[i][att_cpu[i]].tolist() for i in range(bs)]
        t0 = time.perf_counter()
        self.rollout.profile = bool(cfg_get(ro, "log_stats", False))      # rollout.log_stats: per-call prefill / decode / capture timings
        self.rollout.record_routing = bool(cfg_get(ro, "enable_rollout_routing_replay", False))
        self.rollout.wake_up()
        mm = prompts.non_tensor_batch.get("multi_modal_inputs") if prompts.non_tensor_batch else None
        outs = self.rollout.generate(plist, sp, eos_token_id=eos, multi_modal=[(m or None) for m in mm] if mm is not None else None)
        if self.rollout.profile and self.rank == 0:
            print(f"[rollout stats] {self.rollout.stats}", flush=True)
        if bool(cfg_get(ro, "free_cache_engine", True)):
            self.rollout.sleep()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        resp = torch.full((bs, R), pad_id, dtype=ids_cpu.dtype)
        lps = torch.zeros(bs, R, dtype=torch.float32)
        rmask = torch.zeros(bs, R, dtype=att.dtype)
        for i, o in enumerate(outs):
            n = len(o.token_ids)
            resp[i, :n] = torch.tensor(o.token_ids, dtype=ids_cpu.dtype)
            rmask[i, :n] = 1
            if o.log_probs is not None:
                lps[i, :n] = torch.tensor(o.log_probs)
        full_ids = torch.cat([ids_cpu, resp], dim=1)
        full_att = torch.cat([att.cpu(), rmask], dim=1)
        batch = TensorBatch({"prompts": ids_cpu, "responses": resp, "input_ids": full_ids, "attention_mask": full_att,
                             "position_ids": compute_position_id_with_mask(full_att), "response_mask": rmask,
                             "rollout_log_probs": lps}, batch_size=(bs,))
        if self.rollout.record_routing and outs and outs[0].routed_experts is not None:
            # router replay R3: the experts the rollout chose for every token, laid out like input_ids (left-padded prompt,
            # right-padded response); -1 rows (padding) are never read because the trainer packs by the attention mask
            Lr, kr = outs[0].routed_experts.shape[1:]
            routed = torch.full((bs, P + R, Lr, kr), -1, dtype=torch.int16)
            for i, o in enumerate(outs):
                lp_i = int(att_cpu[i].sum())
                rt = torch.from_numpy(np.ascontiguousarray(o.routed_experts))
                routed[i, P - lp_i:P + len(o.token_ids)] = rt
            batch["routed_experts"] = routed
        if sp.top_logprobs > 0:
            # the sampler's top-k head per response token (padding rows: ids 0..k-1 with log-prob -1e4, i.e. zero mass)
            k = sp.top_logprobs
            tids = torch.arange(k).expand(bs, R, k).clone()
            tlps = torch.full((bs, R, k), -1e4, dtype=torch.float32)
            for i, o in enumerate(outs):
                n = len(o.token_ids)
                if n and o.top_ids is not None:
                    tids[i, :n] = torch.tensor(o.top_ids)
                    tlps[i, :n] = torch.tensor(o.top_log_probs)
            batch["rollout_topk_ids"], batch["rollout_topk_log_probs"] = tids, tlps
        n_tok = int(rmask.sum())
        out = DataProto(batch=batch, non_tensor_batch=dict(prompts.non_tensor_batch),
                        meta_info={"timing": {"generate_sequences": dt}, "metrics": [{"rollout/tokens_per_s": n_tok / max(dt, 1e-9)}]})
        return out

    # ------------------------------------------------------------------ log-probs
    def _router_replay_mode(self) -> str:
        """``actor.router_replay.mode``: ``disabled`` | ``R2`` (routing recorded by the old-log-prob pass, replayed by the update)
        | ``R3`` (routing recorded by the rollout engine, replayed by the old-log-prob pass and the update). Reference:
        verl/utils/megatron/router_replay_patch.py:38-165, verl/workers/engine/megatron/transformer_impl.py:871-907,933-971."""
        return str(cfg_get(self.config, "actor.router_replay.mode", "disabled") or "disabled").upper()

    @staticmethod
    def _without_routing(batch):
        if "routed_experts" not in batch:
            return batch
        return TensorBatch({k: v for k, v in batch.items() if k != "routed_experts"}, batch_size=batch.batch_size)

    def _logprob_pass(self, worker: TrainingWorker, data: DataProto, calculate_entropy: bool, replay: bool = False, record: bool = False) -> dict:
        meta = dict(data.meta_info)
        meta["calculate_entropy"] = calculate_entropy
        meta.setdefault("temperature", float(cfg_get(self.config, "rollout.temperature", 1.0)))
        if record:
            meta["record_routing"] = True
        d = DataProto(batch=data.batch if replay else self._without_routing(data.batch), non_tensor_batch=_model_inputs(data), meta_info=meta)
        return worker.infer_batch(d)["model_output"]

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("actor"))
    @_annotate("compute_log_prob", "actor")
    def compute_log_prob(self, data: DataProto) -> DataProto:
        mode = self._router_replay_mode()
        if self.ref is not None and hasattr(self.ref.engine, "prefetch_params") and self.ref.engine.is_param_offload_enabled:
            self.ref.engine.prefetch_params()       # the reference pass comes next: its parked weights travel during this pass
        mo = self._logprob_pass(self.actor, data, calculate_entropy=True, replay=mode == "R3", record=mode == "R2")
        tensors = {"old_log_probs": _to_host(mo["log_probs"])}
        if "entropy" in mo:
            tensors["entropys"] = _to_host(mo["entropy"])
        if mode == "R2" and "routed_experts" in mo:
            tensors["routed_experts"] = _to_host(mo["routed_experts"])
        return DataProto.from_dict(tensors=tensors, meta_info={"temperature": data.meta_info.get("temperature", 1.0)})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("actor"))
    @_annotate("compute_ref_log_prob", "ref")
    def compute_ref_log_prob(self, data: DataProto) -> DataProto:
        worker = self.ref if self.ref is not None else self.actor
        mo = self._logprob_pass(worker, data, calculate_entropy=False)      # the frozen policy routes by itself
        return DataProto.from_dict(tensors={"ref_log_prob": _to_host(mo["log_probs"])})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("actor"))
    def compute_teacher_topk(self, data: DataProto) -> DataProto:
        """Teacher forward over the student's samples: its k most likely tokens and their log-probs per response position."""
        assert self.teacher is not None, "distillation.enable=true is needed for a teacher pass"
        meta = dict(data.meta_info)
        meta["calculate_entropy"] = False
        meta["return_topk"] = int(cfg_get(self.config, "distillation.topk", 32))
        meta["temperature"] = 1.0
        meta.pop("use_prefix_grouper", None)
        d = DataProto(batch=data.batch, non_tensor_batch=_model_inputs(data), meta_info=meta)
        mo = self.teacher.infer_batch(d)["model_output"]
        return DataProto.from_dict(tensors={"teacher_topk_ids": _to_host(mo["topk_ids"]), "teacher_topk_log_probs": _to_host(mo["topk_log_probs"])})

    # ------------------------------------------------------------------ update
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("actor"))
    @_annotate("update_actor", "actor")
    def update_actor(self, data: DataProto) -> DataProto:
        ac = cfg_get(self.config, "actor")
        meta = dict(data.meta_info)
        if self.teacher is not None or getattr(self, "_distill", False):
            meta["distillation"] = True
        meta.setdefault("temperature", float(cfg_get(self.config, "rollout.temperature", 1.0)))
        meta["calculate_entropy"] = bool(cfg_get(ac, "calculate_entropy", False)) or float(cfg_get(ac, "entropy_coeff", 0.0)) != 0.0
        replay = self._router_replay_mode() in ("R2", "R3")
        data = DataProto(batch=data.batch if replay else self._without_routing(data.batch), non_tensor_batch=_model_inputs(data), meta_info=meta)
        metrics = self.actor.train_mini_batch(data)
        return DataProto(batch=None, non_tensor_batch={}, meta_info={"metrics": metrics})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def update_weights(self):
        """Actor → rollout weight hand-off through this worker's :class:`CheckpointEngineManager` (which path runs is
        described there). Returns the seconds it took; the manager keeps the details in ``last_stats``."""
        if getattr(self, "checkpoint_manager", None) is None:
            from verl_b200.checkpoint_engine.manager import CheckpointEngineManager

            self.checkpoint_manager = CheckpointEngineManager(self, cfg_get(self.config, "rollout.checkpoint_engine.backend", "naive"))
        return self.checkpoint_manager.update_weights()["seconds_total"]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        self.actor.engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False):
        self.actor.engine.load_checkpoint(local_path, hdfs_path, del_local_after_load)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def wait_checkpoint(self):
        _wait_checkpoint(self.actor.engine)


class CriticWorker(Worker, _ProfiledWorker):
    """Value model: ``compute_values`` (forward) and ``update_critic`` (clipped value loss)."""

    def __init__(self, config):
        super().__init__()
        ensure_process_group(int(cfg_get(config, "nccl_timeout", 600)))
        self.config = config
        self.critic: Optional[TrainingWorker] = None
        self.profiler = _role_profiler(config, "")

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        self.critic = TrainingWorker(_role_cfg(self.config, "critic", "value_model"), role="critic")
        self.critic.reset()
        self.critic.set_loss_fn(partial(value_loss, self.config))
        eng = self.critic.engine
        self._register_dispatch_collect_info("critic", dp_rank=eng.get_data_parallel_rank(), is_collect=eng.is_mp_src_rank_with_outputs())

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("critic"))
    @_annotate("compute_values", "critic")
    def compute_values(self, data: DataProto) -> DataProto:
        d = DataProto(batch=data.batch, non_tensor_batch=_model_inputs(data), meta_info=dict(data.meta_info))
        mo = self.critic.infer_batch(d)["model_output"]
        vals = mo["values"].cpu() * data.batch["response_mask"].to(mo["values"].dtype).cpu()
        return DataProto.from_dict(tensors={"values": vals})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("critic"))
    @_annotate("update_critic", "critic")
    def update_critic(self, data: DataProto) -> DataProto:
        d = DataProto(batch=data.batch, non_tensor_batch=_model_inputs(data), meta_info=dict(data.meta_info))
        metrics = self.critic.train_mini_batch(d)
        return DataProto(batch=None, non_tensor_batch={}, meta_info={"metrics": metrics})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        self.critic.engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False):
        self.critic.engine.load_checkpoint(local_path, hdfs_path, del_local_after_load)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def wait_checkpoint(self):
        _wait_checkpoint(self.critic.engine)


class RewardModelWorker(Worker):
    """Discriminative reward model: a frozen model with a scalar head scores every (prompt, response) pair; the score of the
    last response token becomes the sequence reward (``rm_scores`` [bs, R], zero elsewhere). Same engines as the critic, forward
    only. Reference: the reward-model server behind the reward loop (``verl/experimental/reward_loop/reward_loop.py:93-343``,
    discriminative ``/classify``-style scoring) and the legacy ``RewardModelWorker``."""

    def __init__(self, config):
        super().__init__()
        ensure_process_group(int(cfg_get(config, "nccl_timeout", 600)))
        self.config = config
        self.rm: Optional[TrainingWorker] = None

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        c = self.config
        strategy = cfg_get(c, "strategy", "fsdp")
        eng = dict(cfg_get(c, "fsdp_config", {}) or {}) if str(strategy).startswith("fsdp") else dict(cfg_get(c, "megatron", {}) or {})
        eng["forward_only"] = True
        model = cfg_get(c, "model", None) or {"path": cfg_get(c, "path", None), "preset": cfg_get(c, "preset", None)}
        mbs = cfg_get(c, "micro_batch_size_per_gpu", None)
        cfg = {"model_type": "value_model", "backend": strategy, "model": model, "engine": eng, "optim": None, "checkpoint": None,
               "log_prob_micro_batch_size_per_gpu": mbs, "ppo_micro_batch_size_per_gpu": mbs,
               "log_prob_use_dynamic_bsz": cfg_get(c, "use_dynamic_bsz", False), "log_prob_max_token_len_per_gpu": cfg_get(c, "forward_max_token_len_per_gpu", None),
               "nccl_timeout": cfg_get(c, "nccl_timeout", 600)}
        self.rm = TrainingWorker(cfg, role="reward_model")
        self.rm.reset()
        e = self.rm.engine
        self._register_dispatch_collect_info("reward_model", dp_rank=e.get_data_parallel_rank(), is_collect=e.is_mp_src_rank_with_outputs())

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("reward_model"))
    def compute_rm_score(self, data: DataProto) -> DataProto:
        d = DataProto(batch=data.batch, non_tensor_batch=_model_inputs(data), meta_info=dict(data.meta_info))
        vals = self.rm.infer_batch(d)["model_output"]["values"].float().cpu()           # [bs, R] head output per response token
        mask = data.batch["response_mask"].cpu()
        last = (mask.sum(-1) - 1).clamp(min=0).long()
        scores = torch.zeros_like(vals)
        rows = torch.arange(vals.shape[0])
        scores[rows, last] = vals[rows, last] * (mask.sum(-1) > 0).to(vals.dtype)
        return DataProto.from_dict(tensors={"rm_scores": scores})
