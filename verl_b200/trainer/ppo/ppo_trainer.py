"""Synchronous PPO / GRPO trainer (single-controller dataflow).

One step: generate → reward → (balance) → old log-prob → ref log-prob → values → advantages (on the controller) →
update critic → update actor → (validate / checkpoint) → weight hand-off → metrics. Parity target:
``verl/trainer/ppo/ray_trainer.py`` (apply_kl_penalty :78, compute_response_mask :120, compute_advantage :187,
RayPPOTrainer.init_workers :772, _validate :596, _save_checkpoint :983, _load_checkpoint :1052, fit :1405-1823).
"""

from __future__ import annotations

import os
import time
import uuid
from collections import defaultdict
from contextlib import contextmanager
from typing import Optional

import numpy as np
import torch

from verl_b200.protocol import DataProto, collate_fn
from verl_b200.single_controller.base import ClassWithInitArgs, ResourcePool
from verl_b200.trainer.ppo import core_algos
from verl_b200.trainer.ppo.core_algos import AdvantageEstimator, agg_loss
from verl_b200.trainer.ppo.metric_utils import (compute_data_metrics, compute_throughout_metrics, compute_timing_metrics,
                                                compute_variance_proxy_metrics, process_validation_metrics, reduce_metrics)
from verl_b200.trainer.ppo.reward import compute_reward, load_reward_manager
from verl_b200.utils import torch_functional as VF
from verl_b200.utils.checkpoint.checkpoint_manager import find_latest_ckpt_path, should_save_ckpt_esi
from verl_b200.utils.seqlen_balancing import calculate_workload, get_seqlen_balanced_partitions, log_seqlen_unbalance
from verl_b200.utils.tracking import Tracking, ValidationGenerationsLogger

__all__ = ["PPOTrainer", "RayPPOTrainer", "apply_kl_penalty", "compute_response_mask", "compute_advantage", "marked_timer"]


@contextmanager
def marked_timer(name: str, timing_raw: dict, **kwargs):
    """Accumulate wall time of a section into ``timing_raw[name]`` (and emit an NVTX range when CUDA is present)."""
    use_nvtx = torch.cuda.is_available()
    if use_nvtx:
        torch.cuda.nvtx.range_push(name)
    t0 = time.perf_counter()
    try:
        yield
    finally:
        timing_raw[name] = timing_raw.get(name, 0.0) + time.perf_counter() - t0
        if use_nvtx:
            torch.cuda.nvtx.range_pop()


def apply_kl_penalty(data: DataProto, kl_ctrl, kl_penalty: str = "kl"):
    """token_level_rewards = token_level_scores − β·KL(π_old ‖ π_ref); updates the adaptive controller."""
    mask = data.batch["response_mask"]
    kld = core_algos.kl_penalty(data.batch["old_log_probs"], data.batch["ref_log_prob"], kl_penalty=kl_penalty) * mask
    beta = kl_ctrl.value
    data.batch["token_level_rewards"] = data.batch["token_level_scores"] - beta * kld
    current_kl = torch.mean(VF.masked_mean(kld, mask=mask, axis=-1), dim=0).item()
    kl_ctrl.update(current_kl=current_kl, n_steps=data.batch["responses"].shape[0])
    return data, {"actor/reward_kl_penalty": current_kl, "actor/reward_kl_penalty_coeff": beta}


def compute_response_mask(data: DataProto) -> torch.Tensor:
    R = data.batch["responses"].size(1)
    return data.batch["attention_mask"][:, -R:]


def compute_advantage(data: DataProto, adv_estimator, gamma: float = 1.0, lam: float = 1.0, num_repeat: int = 1,
                      norm_adv_by_std_in_grpo: bool = True, config=None) -> DataProto:
    if "response_mask" not in data.batch.keys():
        data.batch["response_mask"] = compute_response_mask(data)
    name = adv_estimator.value if isinstance(adv_estimator, AdvantageEstimator) else adv_estimator
    fn = core_algos.get_adv_estimator_fn(name)
    b = data.batch
    kwargs = dict(token_level_rewards=b["token_level_rewards"], response_mask=b["response_mask"], config=config)
    if name == "gae":
        kwargs.update(values=b["values"], gamma=gamma, lam=lam)
    else:
        if "uid" in data.non_tensor_batch:
            kwargs["index"] = data.non_tensor_batch["uid"]
        if name in ("grpo", "grpo_vectorized", "gdpo", "grpo_passk"):
            kwargs["norm_adv_by_std_in_grpo"] = norm_adv_by_std_in_grpo
        if name == "gdpo":
            kwargs.update(non_tensor_batch=data.non_tensor_batch, batch=b)
        if name == "remax":
            kwargs["reward_baselines"] = b["reward_baselines"]
        if name == "reinforce_plus_plus":
            kwargs["gamma"] = gamma
        if name in ("optimal_token_baseline", "tir_optimal_token_baseline"):
            kwargs.update(old_log_probs=b["old_log_probs"], sum_pi_squared=b["sum_pi_squared"],
                          rollout_is_weights=b.get("rollout_is_weights"))
    adv, ret = fn(**kwargs)
    data.batch["advantages"], data.batch["returns"] = adv, ret
    return data


def _g(cfg, key, default=None):
    cur = cfg
    for part in key.split("."):
        if cur is None:
            return default
        cur = cur.get(part) if hasattr(cur, "get") else getattr(cur, part, None)
    return default if cur is None else cur


class PPOTrainer:
    """Controller-side trainer. With the ``spmd`` worker backend every rank runs this same object (torchrun); with the
    ``process`` backend one driver owns spawned workers."""

    def __init__(self, config, tokenizer=None, processor=None, reward_fn=None, val_reward_fn=None, train_dataset=None,
                 val_dataset=None, collate=None, train_sampler=None, device_name: Optional[str] = None):
        self.config = config
        self.tokenizer = tokenizer
        self.processor = processor
        self.device_name = device_name or _g(config, "trainer.device", "cuda")
        self.reward_fn = reward_fn
        self.val_reward_fn = val_reward_fn
        self.collate = collate or collate_fn
        adv = _g(config, "algorithm.adv_estimator", "gae")
        self.use_critic = _g(config, "critic.enable", None)
        if self.use_critic is None:
            self.use_critic = adv == "gae"
        self.use_reference_policy = bool(_g(config, "algorithm.use_kl_in_reward", False)) or bool(_g(config, "actor_rollout_ref.actor.use_kl_loss", False))
        self.kl_ctrl_in_reward = core_algos.get_kl_controller(config.algorithm.kl_ctrl) if _g(config, "algorithm.use_kl_in_reward", False) else None
        self.n_gpus = int(_g(config, "trainer.n_gpus_per_node", 1)) * int(_g(config, "trainer.nnodes", 1))
        self.global_steps = 0
        self.validation_generations_logger = ValidationGenerationsLogger(_g(config, "trainer.project_name"), _g(config, "trainer.experiment_name"))
        self._create_dataloader(train_dataset, val_dataset, train_sampler)

    # ------------------------------------------------------------------ data
    def _create_dataloader(self, train_dataset, val_dataset, train_sampler):
        from torch.utils.data import DataLoader

        from verl_b200.utils.dataset import create_rl_dataset, create_rl_sampler

        dc = self.config.data
        if dc.get("vision") is None:
            # vision-language actor: the dataset needs the tower geometry (patch / merge sizes, placeholder ids) to cut images
            mc = self.config.actor_rollout_ref.model
            vis = None
            if mc.get("preset"):
                from verl_b200.models.config import PRESETS

                vis = PRESETS[mc.get("preset")].vision
            elif mc.get("path") and os.path.exists(os.path.join(os.path.expanduser(str(mc.get("path"))), "config.json")):
                from verl_b200.models.config import ModelConfig

                vis = ModelConfig.from_pretrained(os.path.expanduser(str(mc.get("path")))).vision
            if vis:
                dc["vision"] = dict(vis)
        if train_dataset is None:
            train_dataset = create_rl_dataset(dc.get("train_files"), dc, self.tokenizer, self.processor, is_train=True)
        if val_dataset is None and (dc.get("val_files") or _g(dc, "synthetic.enable", False)):
            val_dataset = create_rl_dataset(dc.get("val_files"), dc, self.tokenizer, self.processor, is_train=False)
        self.train_dataset, self.val_dataset = train_dataset, val_dataset
        if train_sampler is None:
            train_sampler = create_rl_sampler(dc, train_dataset)
        try:
            from torchdata.stateful_dataloader import StatefulDataLoader as Loader
        except Exception:  # noqa: BLE001
            Loader = DataLoader
        self.train_dataloader = Loader(train_dataset, batch_size=int(dc.get("gen_batch_size", dc.train_batch_size)), num_workers=int(dc.get("dataloader_num_workers", 0)),
                                       drop_last=True, collate_fn=self.collate, sampler=train_sampler)
        self.val_dataloader = None
        if val_dataset is not None:
            vbs = dc.get("val_batch_size") or len(val_dataset)
            self.val_dataloader = Loader(val_dataset, batch_size=int(vbs), num_workers=0, shuffle=False, drop_last=False, collate_fn=self.collate)
        total = len(self.train_dataloader) * int(_g(self.config, "trainer.total_epochs", 1))
        if _g(self.config, "trainer.total_training_steps") is not None:
            total = int(self.config.trainer.total_training_steps)
        self.total_training_steps = total
        self.config.actor_rollout_ref.actor.optim["total_training_steps"] = total
        if "critic" in self.config and self.config.critic.get("optim") is not None:
            self.config.critic.optim["total_training_steps"] = total

    # ------------------------------------------------------------------ workers
    def init_workers(self):
        from verl_b200.workers.engine_workers import ActorRolloutRefWorker, CriticWorker, RewardModelWorker

        backend = _g(self.config, "trainer.worker_backend", "spmd")
        role = "actor_rollout_ref" if self.use_reference_policy else "actor_rollout"
        arr = ClassWithInitArgs(ActorRolloutRefWorker, config=self.config.actor_rollout_ref, role=role)
        if self.use_critic:
            # the critic's mini-batch is counted in prompts like the actor's; its worker needs n to turn it into trajectories
            self.config.critic["rollout_n"] = int(_g(self.config, "actor_rollout_ref.rollout.n", 1))
        crit = ClassWithInitArgs(CriticWorker, config=self.config.critic) if self.use_critic else None
        if backend == "spmd":
            from verl_b200.single_controller.spmd import SPMDWorkerGroup, init_spmd_process_group

            init_spmd_process_group(int(_g(self.config, "actor_rollout_ref.nccl_timeout", 600)))
            self.actor_rollout_wg = SPMDWorkerGroup(cls_with_init_args=arr)
            self.critic_wg = SPMDWorkerGroup(cls_with_init_args=crit) if crit is not None else None
        elif backend == "process":
            from verl_b200.single_controller.process import ProcessWorkerGroup, create_colocated_worker_cls

            pool = ResourcePool([int(self.config.trainer.n_gpus_per_node)] * int(self.config.trainer.nnodes))
            class_dict = {"actor_rollout": arr}
            if crit is not None:
                class_dict["critic"] = crit
            wg = ProcessWorkerGroup(pool, create_colocated_worker_cls(class_dict), use_gpu=self.device_name == "cuda")
            views = wg.spawn(set(class_dict))
            self._root_wg = wg
            self.actor_rollout_wg = views["actor_rollout"]
            self.critic_wg = views.get("critic")
            wg.start_worker_aliveness_check(1.0)
        else:
            raise ValueError(f"unknown trainer.worker_backend {backend}")
        self.ref_policy_wg = self.actor_rollout_wg
        self.rm_wg = None
        if bool(_g(self.config, "reward.reward_model.enable", False)):
            # a frozen scalar-head model scores the samples; rule rewards (if any) are added on top
            if backend != "spmd":
                raise NotImplementedError("the reward-model worker runs on the spmd backend")
            from verl_b200.single_controller.spmd import SPMDWorkerGroup

            self.rm_wg = SPMDWorkerGroup(cls_with_init_args=ClassWithInitArgs(RewardModelWorker, config=self.config.reward.reward_model))
            self.rm_wg.init_model()
        if self.critic_wg is not None:
            self.critic_wg.init_model()
        self.actor_rollout_wg.init_model()
        self.actor_rollout_wg.update_weights()

    # ------------------------------------------------------------------ checkpoint
    def _save_checkpoint(self):
        root = os.path.expanduser(self.config.trainer.default_local_dir)
        step_dir = os.path.join(root, f"global_step_{self.global_steps}")
        print(f"local_global_step_folder: {step_dir}")
        self._finish_pending_checkpoint(block=True)          # an earlier asynchronous save gets its tracker entry first
        self.actor_rollout_wg.save_checkpoint(os.path.join(step_dir, "actor"), None, self.global_steps, _g(self.config, "trainer.max_actor_ckpt_to_keep"))
        if self.use_critic:
            self.critic_wg.save_checkpoint(os.path.join(step_dir, "critic"), None, self.global_steps, _g(self.config, "trainer.max_critic_ckpt_to_keep"))
        rank = int(os.environ.get("RANK", "0")) if _g(self.config, "trainer.worker_backend", "spmd") == "spmd" else 0
        if rank == 0:
            os.makedirs(step_dir, exist_ok=True)
            if hasattr(self.train_dataloader, "state_dict"):
                torch.save(self.train_dataloader.state_dict(), os.path.join(step_dir, "data.pt"))
        # the tracker names a step only once all of its files exist: right away for synchronous saves, after every rank's
        # background writer has dropped its marker for asynchronous ones (polled after each step, awaited at the end of fit)
        self._pending_ckpt = (root, step_dir, self.global_steps)
        self._pending_ckpt_tracked = False
        asynchronous = bool(_g(self.config, "actor_rollout_ref.actor.checkpoint.async_save", False)) or bool(_g(self.config, "critic.checkpoint.async_save", False))
        self._finish_pending_checkpoint(block=not asynchronous)

    def _finish_pending_checkpoint(self, block: bool) -> bool:
        """Write ``latest_checkpointed_iteration.txt`` for the last save once all of its writers are done.

        ``block=False`` only looks at the marker files (no collective; ranks may see different answers, so nothing but the
        tracker file changes). ``block=True`` is collective: every controller joins the writers, then the entry is closed."""
        from verl_b200.utils.checkpoint.checkpoint_manager import BaseCheckpointManager as M

        pend = getattr(self, "_pending_ckpt", None)
        if pend is None:
            return True
        root, step_dir, step = pend
        roles = ["actor"] + (["critic"] if self.use_critic else [])
        if block:
            self.actor_rollout_wg.wait_checkpoint()
            if self.use_critic:
                self.critic_wg.wait_checkpoint()
        world = max(1, self.actor_rollout_wg.world_size)
        rank = int(os.environ.get("RANK", "0")) if _g(self.config, "trainer.worker_backend", "spmd") == "spmd" else 0
        done = all(M.async_save_complete(os.path.join(step_dir, r), world) for r in roles)
        if block and not done:
            raise RuntimeError(f"checkpoint writers finished but {step_dir} is incomplete")
        if done and rank == 0 and not getattr(self, "_pending_ckpt_tracked", False):
            tmp = os.path.join(root, "latest_checkpointed_iteration.txt.tmp")
            with open(tmp, "w") as f:
                f.write(str(step))
            os.replace(tmp, os.path.join(root, "latest_checkpointed_iteration.txt"))
            self._pending_ckpt_tracked = True
        if block:
            if rank == 0:
                for r in roles:
                    M.finish_async_save(os.path.join(step_dir, r), world)
            self._pending_ckpt = None
            self._pending_ckpt_tracked = False
        return done

    def _load_checkpoint(self) -> int:
        mode = _g(self.config, "trainer.resume_mode", "auto")
        if mode == "disable":
            return 0
        root = os.path.expanduser(self.config.trainer.default_local_dir)
        if mode == "resume_path":
            step_dir = _g(self.config, "trainer.resume_from_path")
            assert step_dir and "global_step_" in step_dir, "resume_from_path must point at a global_step_N folder"
        else:
            step_dir = find_latest_ckpt_path(root)
        if step_dir is None:
            print("Training from scratch")
            return 0
        self.global_steps = int(str(step_dir).rstrip("/").split("global_step_")[-1])
        print(f"Resuming from {step_dir} (global step {self.global_steps})")
        self.actor_rollout_wg.load_checkpoint(os.path.join(step_dir, "actor"), None, bool(_g(self.config, "trainer.del_local_ckpt_after_load", False)))
        if self.use_critic:
            self.critic_wg.load_checkpoint(os.path.join(step_dir, "critic"), None, False)
        data_pt = os.path.join(step_dir, "data.pt")
        if os.path.exists(data_pt) and hasattr(self.train_dataloader, "load_state_dict"):
            self.train_dataloader.load_state_dict(torch.load(data_pt, weights_only=False))
        return self.global_steps

    # ------------------------------------------------------------------ helpers
    def _balance_batch(self, batch: DataProto, metrics: dict, logging_prefix: str = "global_seqlen"):
        """Reorder samples so that each data-parallel rank's contiguous chunk carries an equal attention+MLP workload."""
        lens = batch.batch["attention_mask"].view(len(batch), -1).sum(-1)
        world = self.actor_rollout_wg.world_size
        if world <= 1 or len(batch) % world != 0:
            return
        uid = batch.non_tensor_batch.get("uid") if _g(self.config, "actor_rollout_ref.actor.use_prefix_grouper", False) else None
        if uid is not None:
            # prefix sharing: the samples of one prompt stay on one rank (reference: group-level balancing,
            # verl/trainer/ppo/ray_trainer.py:1185-1240); whole groups are balanced instead of single samples
            groups: dict = {}
            for i, u in enumerate(uid.tolist()):
                groups.setdefault(u, []).append(i)
            members = list(groups.values())
            if len(members) % world == 0 and len({len(m) for m in members}) == 1:
                work = [float(sum(calculate_workload(lens[m]).tolist())) for m in members]
                gparts = get_seqlen_balanced_partitions(work, world, equal_size=True)
                parts = [[i for g in gp for i in members[g]] for gp in gparts]
                batch.reorder(torch.tensor([i for p in parts for i in p]))
                metrics.update(log_seqlen_unbalance(lens.tolist(), parts, logging_prefix))
                return
        parts = get_seqlen_balanced_partitions(calculate_workload(lens).tolist(), world, equal_size=True)
        for p in parts:   # shortest-first inside a rank keeps micro-batches homogeneous
            p.sort(key=lambda i: int(lens[i]))
        batch.reorder(torch.tensor([i for p in parts for i in p]))
        metrics.update(log_seqlen_unbalance(lens.tolist(), parts, logging_prefix))

    def _num_experts(self) -> Optional[int]:
        """Experts per MoE layer of the actor's architecture (preset or ``config.json``), for the load-balance metrics."""
        mc = self.config.actor_rollout_ref.model
        try:
            if mc.get("preset"):
                from verl_b200.models.config import PRESETS

                return int(PRESETS[mc.get("preset")].num_experts) or None
            if mc.get("path"):
                from verl_b200.models.config import ModelConfig

                return int(ModelConfig.from_pretrained(os.path.expanduser(str(mc.get("path")))).num_experts) or None
        except Exception:  # noqa: BLE001
            return None
        return None

    def _gen_meta(self, validate: bool = False) -> dict:
        tk = self.tokenizer
        return {"eos_token_id": getattr(tk, "eos_token_id", None) if tk is not None else _g(self.config, "data.eos_token_id"),
                "pad_token_id": (getattr(tk, "pad_token_id", 0) if tk is not None else 0) or 0,
                "do_sample": not validate or bool(_g(self.config, "actor_rollout_ref.rollout.val_kwargs.do_sample", False)),
                "validate": validate, "global_steps": self.global_steps,
                "response_length": int(self.config.data.max_response_length)}

    def _dump_generations(self, batch: DataProto, scores: list, extra: dict, dump_dir: str, append: bool = False) -> str:
        """One JSON line per trajectory in ``{dump_dir}/{global_step}.jsonl``: prompt and response (text when a tokenizer is
        known, token ids otherwise), score, ground truth, data source and the scalar extras of the reward function
        (reference: ``verl/trainer/ppo/ray_trainer.py:479-545``, ``trainer.rollout_data_dir`` / ``validation_data_dir``)."""
        import json

        os.makedirs(dump_dir, exist_ok=True)
        fn = os.path.join(dump_dir, f"{self.global_steps}.jsonl")
        b, nt = batch.batch, batch.non_tensor_batch
        P = b["prompts"].shape[1]
        tok = self.tokenizer

        def text(ids):
            ids = [int(t) for t in ids]
            return tok.decode(ids, skip_special_tokens=False) if tok is not None else ids

        with open(fn, "a" if append else "w") as f:
            for i in range(len(batch)):
                pm, rm = b["attention_mask"][i, :P].bool(), b["attention_mask"][i, P:].bool()
                row = {"input": text(b["prompts"][i][pm]), "output": text(b["responses"][i][rm]), "score": float(scores[i]), "step": int(self.global_steps),
                       "data_source": str(nt["data_source"][i]) if "data_source" in nt else None}
                rmeta = nt["reward_model"][i] if "reward_model" in nt else None
                if isinstance(rmeta, dict) and "ground_truth" in rmeta:
                    row["gts"] = rmeta["ground_truth"] if isinstance(rmeta["ground_truth"], (str, int, float, list)) else str(rmeta["ground_truth"])
                for k, v in (extra or {}).items():
                    if len(v) == len(batch) and isinstance(v[i], (str, int, float, bool)):
                        row[k] = v[i]
                f.write(json.dumps(row, ensure_ascii=False) + "\n")
        return fn

    def _served_teacher_topk(self, batch: DataProto) -> DataProto:
        """Top-k heads of teachers that run on rollout servers of their own (``distillation.teacher_mode=server``): servers listed in
        ``distillation.teacher_addresses`` ({routing key: [host:port, ...]}) are used as they are, otherwise one fleet per entry of
        ``distillation.teacher_models`` is started on ``distillation.teacher_devices``. Samples are routed by
        ``distillation.teacher_key`` of their non-tensor data when several teachers exist."""
        from verl_b200.experimental.teacher_loop import AsyncTeacherLLMServerManager, build_teacher_fleet
        from verl_b200.workers.rollout.llm_server import LLMServerClient

        d = _g(self.config, "actor_rollout_ref.distillation", {})
        if getattr(self, "_teacher_mgr", None) is None:
            addrs = dict(_g(d, "teacher_addresses", None) or {})
            if addrs:
                clients = {k: LLMServerClient({f"{k}-{i}": a for i, a in enumerate(v if isinstance(v, (list, tuple)) else [v])}) for k, v in addrs.items()}
                self._teacher_fleet = {}
            else:
                models = dict(_g(d, "teacher_models", None) or {})
                if not models:
                    tm = _g(d, "teacher_model", {}) or {}
                    models = {"default": {"model_path": tm.get("path") or tm.get("preset")}}
                devs = _g(d, "teacher_devices", None)
                n = sum(int((m.get("num_replicas", 1) if hasattr(m, "get") else 1) or 1) for m in models.values())
                devs = [None] * n if devs in (None, "", []) else [str(x) for x in (devs if isinstance(devs, (list, tuple)) else str(devs).split(","))]
                self._teacher_fleet = build_teacher_fleet(models, devs, int(_g(d, "n_gpus_per_node", 8) or 8), _g(self.config, "actor_rollout_ref.rollout", None))
                clients = {k: m.client() for k, m in self._teacher_fleet.items()}
            self._teacher_mgr = AsyncTeacherLLMServerManager({"teacher_key": _g(d, "teacher_key", "data_source"), "topk": int(_g(d, "topk", 32)),
                                                              "teacher_models": {k: {} for k in clients}}, clients)
        mgr = self._teacher_mgr
        keys = None
        if len(mgr.teacher_client) > 1:
            col = batch.non_tensor_batch.get(mgr.teacher_key)
            if col is None:
                raise ValueError(f"multi-teacher distillation routes by {mgr.teacher_key!r}, which the batch does not carry")
            keys = [str(x) for x in col]
        ids, lps = mgr.compute_teacher_topk(batch.batch["prompts"], batch.batch["responses"], batch.batch["attention_mask"], keys,
                                            int(getattr(self.tokenizer, "pad_token_id", 0) or 0))
        return DataProto.from_dict(tensors={"teacher_topk_ids": ids, "teacher_topk_log_probs": lps})

    def _validate(self) -> dict:
        if self.val_dataloader is None or self.val_reward_fn is None:
            return {}
        scores, sources, uids = [], [], []
        extra_all = defaultdict(list)
        n = int(_g(self.config, "actor_rollout_ref.rollout.val_kwargs.n", 1))
        for test_data in self.val_dataloader:
            tb = DataProto.from_single_dict(test_data)
            tb.non_tensor_batch["uid"] = np.array([str(uuid.uuid4()) for _ in range(len(tb))], dtype=object)
            tb = tb.repeat(n, interleave=True)
            gen = tb.select(batch_keys=["input_ids", "attention_mask", "position_ids"],
                            non_tensor_batch_keys=[k for k in ("multi_modal_inputs",) if k in tb.non_tensor_batch])
            gen.meta_info = self._gen_meta(validate=True)
            gen, pad = _pad_to(gen, self.actor_rollout_wg.world_size)
            out = self.actor_rollout_wg.generate_sequences(gen)
            out = out[: len(out) - pad] if pad else out
            tb = tb.union(out.select(batch_keys=["prompts", "responses", "response_mask"], non_tensor_batch_keys=[]))
            tb.batch["attention_mask"] = out.batch["attention_mask"]
            tb.batch["input_ids"] = out.batch["input_ids"]
            r, extra = compute_reward(tb, self.val_reward_fn)
            if _g(self.config, "trainer.validation_data_dir", None):
                self._dump_generations(tb, r.sum(-1).tolist(), extra, _g(self.config, "trainer.validation_data_dir"), append=len(scores) > 0)
            scores.extend(r.sum(-1).tolist())
            for k, v in extra.items():
                extra_all[k].extend(v)
            sources.extend(tb.non_tensor_batch.get("data_source", np.array(["unknown"] * len(tb), dtype=object)).tolist())
            uids.extend(tb.non_tensor_batch["uid"].tolist())
        infos = {"reward": scores, **{k: v for k, v in extra_all.items() if len(v) == len(scores)}}
        res = process_validation_metrics(sources, uids, infos)
        metrics = {}
        for src, var2m in res.items():
            core = "acc" if "acc" in var2m else "reward"
            for var, m2v in var2m.items():
                n_max = max(int(name.split("@")[-1].split("/")[0]) for name in m2v)
                for name, val in m2v.items():
                    sec = "val-core" if var == core and any(name.startswith(p) for p in ("mean", "maj", "best")) and f"@{n_max}" in name else "val-aux"
                    metrics[f"{sec}/{src}/{var}/{name}"] = val
        return metrics

    # ------------------------------------------------------------------ the RL step
    def step(self, batch_dict: dict) -> dict:
        """One full RL step on a batch of prompts; returns the step's metrics."""
        cfg = self.config
        metrics: dict = {}
        timing_raw: dict = {}
        batch = DataProto.from_single_dict(batch_dict)
        n = int(cfg.actor_rollout_ref.rollout.n)
        batch.non_tensor_batch["uid"] = np.array([str(uuid.uuid4()) for _ in range(len(batch))], dtype=object)
        with marked_timer("step", timing_raw):
            mm_keys = [k for k in ("multi_modal_inputs",) if k in batch.non_tensor_batch]      # image inputs of vision-language prompts
            gen_batch = batch.select(batch_keys=["input_ids", "attention_mask", "position_ids"], non_tensor_batch_keys=mm_keys)
            gen_batch.meta_info = self._gen_meta()
            gen_batch = gen_batch.repeat(repeat_times=n, interleave=True)
            with marked_timer("gen", timing_raw):
                gen_out = self.actor_rollout_wg.generate_sequences(gen_batch)
                timing_raw.update({f"gen/{k}": float(np.max(v)) if isinstance(v, list) else v
                                   for k, v in (gen_out.meta_info.pop("timing", {}) or {}).items()})
                ro_metrics = gen_out.meta_info.pop("metrics", None)
                if ro_metrics:
                    metrics.update(reduce_metrics(ro_metrics if isinstance(ro_metrics, dict) else {}))
            if cfg.algorithm.adv_estimator == "remax":
                with marked_timer("gen_max", timing_raw):
                    base = batch.select(batch_keys=["input_ids", "attention_mask", "position_ids"], non_tensor_batch_keys=mm_keys)
                    base.meta_info = {**self._gen_meta(), "do_sample": False}
                    base_out = self.actor_rollout_wg.generate_sequences(base)
                    tmp = batch.union(base_out.select(batch_keys=["prompts", "responses", "input_ids", "attention_mask", "position_ids", "response_mask"]))
                    rb, _ = compute_reward(tmp, self.reward_fn)
                    batch.pop(batch_keys=[k for k in base_out.batch.keys() if k in batch.batch.keys() and k not in ("input_ids", "attention_mask", "position_ids")])
                    batch.batch["reward_baselines"] = rb.sum(-1)
            batch = batch.repeat(repeat_times=n, interleave=True)
            batch.pop(batch_keys=["input_ids", "attention_mask", "position_ids"])
            for k in mm_keys:
                gen_out.non_tensor_batch.pop(k, None)      # the repeated batch already holds them
            batch = batch.union(gen_out)
            metrics.update(self.train_on_rollouts(batch, timing_raw, n))
        metrics.update(compute_timing_metrics(batch=self._last_batch, timing_raw=timing_raw))
        metrics.update(compute_throughout_metrics(batch=self._last_batch, timing_raw=timing_raw, n_gpus=max(1, self.actor_rollout_wg.world_size)))
        return metrics

    def train_on_rollouts(self, batch: DataProto, timing_raw: dict, n: int) -> dict:
        """Everything of an RL step after generation: reward, old/ref log-probs, values, advantages, critic and actor updates,
        weight hand-off. ``batch`` holds prompts joined with their rollouts (one row per trajectory, ``uid`` marks the
        prompt group). Returns the metrics; timings go to ``timing_raw``. Shared by the v0 step and the v1 trainers."""
        cfg = self.config
        metrics: dict = {}
        with marked_timer("train", timing_raw):
            if "response_mask" not in batch.batch.keys():
                batch.batch["response_mask"] = compute_response_mask(batch)
            if _g(cfg, "trainer.balance_batch", True):
                self._balance_batch(batch, metrics)
            batch.meta_info["global_token_num"] = torch.sum(batch.batch["attention_mask"], dim=-1).tolist()
            batch.meta_info["temperature"] = float(cfg.actor_rollout_ref.rollout.temperature)
            with marked_timer("reward", timing_raw):
                reward_tensor, reward_extra = compute_reward(batch, self.reward_fn)
                if getattr(self, "rm_wg", None) is not None:
                    rm = self.rm_wg.compute_rm_score(batch).batch["rm_scores"]
                    metrics["reward_model/score_mean"] = float(rm.sum(-1).mean())
                    reward_tensor = reward_tensor + rm.to(reward_tensor.dtype) if bool(_g(cfg, "reward.reward_model.add_rule_reward", True)) else rm.to(reward_tensor.dtype)
            rc = cfg.algorithm.get("rollout_correction") or {}
            bypass = bool(rc.get("bypass_mode", False))
            if bypass:
                from verl_b200.trainer.ppo.rollout_corr_helper import apply_bypass_mode

                apply_bypass_mode(batch, rc, cfg.actor_rollout_ref.actor.policy_loss)
            else:
                with marked_timer("old_log_prob", timing_raw):
                    old = self.actor_rollout_wg.compute_log_prob(batch)
                    ent = old.batch.pop("entropys") if "entropys" in old.batch.keys() else None
                    if ent is not None:
                        ea = agg_loss(ent, batch.batch["response_mask"].float(), cfg.actor_rollout_ref.actor.get("loss_agg_mode", "token-mean"))
                        metrics["actor/entropy"] = ea.item()
                    batch = batch.union(old)
                    if "rollout_log_probs" in batch.batch.keys():
                        from verl_b200.utils.debug.metrics import calculate_debug_metrics

                        metrics.update(calculate_debug_metrics(batch))
            if self.use_reference_policy:
                with marked_timer("ref", timing_raw):
                    batch = batch.union(self.ref_policy_wg.compute_ref_log_prob(batch))
            if bool(_g(cfg, "actor_rollout_ref.distillation.enable", False)):
                with marked_timer("teacher", timing_raw):
                    if str(_g(cfg, "actor_rollout_ref.distillation.teacher_mode", "colocated")) == "server":
                        batch = batch.union(self._served_teacher_topk(batch))
                    else:
                        batch = batch.union(self.actor_rollout_wg.compute_teacher_topk(batch))
            if self.use_critic:
                with marked_timer("values", timing_raw):
                    batch = batch.union(self.critic_wg.compute_values(batch))
            with marked_timer("adv", timing_raw):
                batch.batch["token_level_scores"] = reward_tensor
                if _g(cfg, "trainer.rollout_data_dir", None):
                    self._dump_generations(batch, reward_tensor.sum(-1).tolist(), reward_extra, _g(cfg, "trainer.rollout_data_dir"))
                if reward_extra:
                    batch.non_tensor_batch.update({k: np.array(v, dtype=object) for k, v in reward_extra.items() if len(v) == len(batch)})
                if cfg.algorithm.get("use_kl_in_reward", False):
                    batch, kl_m = apply_kl_penalty(batch, self.kl_ctrl_in_reward, cfg.algorithm.kl_penalty)
                    metrics.update(kl_m)
                else:
                    batch.batch["token_level_rewards"] = batch.batch["token_level_scores"]
                if not bypass and (rc.get("rollout_is") or rc.get("rollout_rs")) and "rollout_log_probs" in batch.batch.keys():
                    from verl_b200.trainer.ppo.rollout_corr_helper import compute_rollout_correction_and_add_to_batch

                    batch, is_m = compute_rollout_correction_and_add_to_batch(batch, rc)
                    metrics.update(is_m)
                batch = compute_advantage(batch, cfg.algorithm.adv_estimator, gamma=cfg.algorithm.gamma, lam=cfg.algorithm.lam, num_repeat=n,
                                          norm_adv_by_std_in_grpo=cfg.algorithm.get("norm_adv_by_std_in_grpo", True), config=cfg.algorithm)
                if cfg.algorithm.get("use_pf_ppo", False):
                    batch = core_algos.compute_pf_ppo_reweight_data(batch, cfg.algorithm.pf_ppo.reweight_method, cfg.algorithm.pf_ppo.weight_pow)
            if self.use_critic:
                with marked_timer("update_critic", timing_raw):
                    co = self.critic_wg.update_critic(batch)
                metrics.update(reduce_metrics(co.meta_info["metrics"]))
            if int(_g(cfg, "trainer.critic_warmup", 0)) <= self.global_steps:
                with marked_timer("update_actor", timing_raw):
                    batch.meta_info["multi_turn"] = bool(_g(cfg, "actor_rollout_ref.rollout.multi_turn.enable", False))
                    if rc.get("score_centering", False):
                        # the update pass also evaluates the sampler's top-k head (rollout.topk_log_probs) under the trainer
                        if not bypass or rc.get("loss_type", "ppo_clip") != "reinforce" or "rollout_topk_ids" not in batch.batch.keys():
                            raise ValueError("score centering needs rollout_correction.bypass_mode=true, loss_type=reinforce and "
                                             "actor_rollout_ref.rollout.topk_log_probs > 0")
                        batch.meta_info.update({"score_centering": True, "rollout_is": rc.get("rollout_is"),
                                                "rollout_is_threshold": rc.get("rollout_is_threshold", 2.0)})
                    ao = self.actor_rollout_wg.update_actor(batch)
                metrics.update(reduce_metrics(ao.meta_info["metrics"]))
            with marked_timer("update_weights", timing_raw):
                self.actor_rollout_wg.update_weights()
        metrics.update(compute_data_metrics(batch=batch, use_critic=self.use_critic))
        metrics.update(compute_variance_proxy_metrics(batch, metrics.get("actor/grad_norm")))
        lb_every = int(_g(cfg, "trainer.moe_lb_metrics_interval", 0) or 0)
        if lb_every > 0 and "routed_experts" in batch.batch.keys():
            from verl_b200.trainer.ppo.metric_utils import RolloutMoELoadBalanceMetricsAccumulator, compute_moe_lb_metrics

            if getattr(self, "_moe_lb", None) is None:
                self._moe_lb = RolloutMoELoadBalanceMetricsAccumulator(int(batch.meta_info.get("num_experts", 0)) or self._num_experts())
            metrics.update(compute_moe_lb_metrics(batch, lb_every, self.global_steps, self._moe_lb))
        nt = batch.non_tensor_batch
        if "spec_num_draft_tokens" in nt:
            from verl_b200.trainer.ppo.metric_utils import compute_spec_decode_metrics

            metrics.update(compute_spec_decode_metrics(nt.get("spec_num_draft_tokens"), nt.get("spec_num_accepted_tokens"), nt.get("spec_num_verify_steps")))
        self._last_batch = batch
        return metrics

    def _profiled_groups(self) -> list:
        groups = [getattr(self, n, None) for n in ("actor_rollout_wg", "ref_policy_wg", "critic_wg", "rm_wg")]
        out = []
        for g in groups:
            if g is not None and hasattr(g, "start_profile") and all(g is not o for o in out):
                out.append(g)
        return out

    def _start_profiling(self) -> None:
        for g in self._profiled_groups():
            g.start_profile(role="e2e", profile_step=self.global_steps)

    def _stop_profiling(self) -> None:
        for g in self._profiled_groups():
            g.stop_profile()

    def fit(self):
        cfg = self.config
        is_main = int(os.environ.get("RANK", "0")) == 0 or _g(cfg, "trainer.worker_backend", "spmd") != "spmd"
        logger = Tracking(cfg.trainer.project_name, cfg.trainer.experiment_name, cfg.trainer.logger if is_main else [],
                          config=dict(cfg)) if is_main else None
        self.global_steps = 0
        if self._load_checkpoint():
            # rollout replicas that keep their own copy of the weights (tensor-parallel shards, ZeRO-3 / TPxPP trainers) were
            # filled before the load: hand the restored weights over before the first validation or rollout
            # (reference: verl/trainer/ppo/ray_trainer.py:1429-1430)
            self.actor_rollout_wg.update_weights()
        if self.val_reward_fn is not None and _g(cfg, "trainer.val_before_train", True):
            val = self._validate()
            if val and logger:
                logger.log(data=val, step=self.global_steps)
            if _g(cfg, "trainer.val_only", False):
                return
        self.global_steps += 1
        last_val = None
        max_step_time = 0.0
        prof_steps = {int(x) for x in (_g(cfg, "global_profiler.steps", None) or [])}
        prof_continuous = bool(_g(cfg, "global_profiler.profile_continuous_steps", False))
        profiling = False
        for epoch in range(int(cfg.trainer.total_epochs)):
            for batch_dict in self.train_dataloader:
                t0 = time.perf_counter()
                is_last = self.global_steps >= self.total_training_steps
                # the steps listed in global_profiler.steps are bracketed by start/stop on every worker group; consecutive listed
                # steps share one capture when profile_continuous_steps is set (reference: verl/trainer/ppo/ray_trainer.py:1119-1152)
                if self.global_steps in prof_steps and not profiling:
                    self._start_profiling()
                    profiling = True
                metrics = self.step(batch_dict)
                if profiling and (is_last or not (prof_continuous and (self.global_steps + 1) in prof_steps)):
                    self._stop_profiling()
                    profiling = False
                max_step_time = max(max_step_time, time.perf_counter() - t0)
                test_freq = int(_g(cfg, "trainer.test_freq", -1))
                if self.val_reward_fn is not None and test_freq > 0 and (is_last or self.global_steps % test_freq == 0):
                    last_val = self._validate()
                    metrics.update(last_val)
                save_freq = int(_g(cfg, "trainer.save_freq", -1))
                esi = should_save_ckpt_esi(max_step_time, redundant_time=float(_g(cfg, "trainer.esi_redundant_time", 0)))
                if save_freq > 0 and (is_last or self.global_steps % save_freq == 0 or esi):
                    if esi:
                        print("Force saving checkpoint: the announced capacity expiry is near.")
                    self._save_checkpoint()
                self._finish_pending_checkpoint(block=False)
                metrics.update({"training/global_step": self.global_steps, "training/epoch": epoch})
                if logger:
                    logger.log(data=metrics, step=self.global_steps)
                self.global_steps += 1
                if is_last:
                    self._finish_pending_checkpoint(block=True)
                    if last_val:
                        print(f"Final validation metrics: {last_val}")
                    return
        self._finish_pending_checkpoint(block=True)


def _pad_to(data: DataProto, divisor: int):
    from verl_b200.protocol import pad_dataproto_to_divisor

    return pad_dataproto_to_divisor(data, divisor)


RayPPOTrainer = PPOTrainer
