"""Supervised fine-tuning on the same engine contract as RL (``torchrun -m verl_b200.trainer.sft_trainer key=value``).

Each sample is a (prompt, response) pair laid out like an RL batch — prompt left-padded, response right-padded — so the
engines' packed forward, fused lm_head log-prob kernel and micro-batching are reused unchanged; the loss is the
token-mean negative log-likelihood over response tokens. Parity target: ``verl/trainer/sft_trainer.py:50-452`` with
``config/sft_trainer_engine.yaml`` keys (data.*, model.*, optim.*, engine.*, trainer.*).
"""

from __future__ import annotations

import os
import sys
import time
from functools import partial

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, Dataset, DistributedSampler

from verl_b200.protocol import DataProto, collate_fn
from verl_b200.utils import torch_functional as VF
from verl_b200.utils.config import Config, apply_overrides, resolve_interpolations
from verl_b200.utils.tracking import Tracking
from verl_b200.workers.engine.base import EngineRegistry
from verl_b200.workers.engine_workers import ensure_process_group
from verl_b200.workers.utils.losses import sft_loss

DEFAULT_CONFIG = {
    "data": {"train_files": None, "val_files": None, "prompt_key": "prompt", "response_key": "response", "max_prompt_length": 256,
             "max_response_length": 256, "train_batch_size": 32, "micro_batch_size_per_gpu": 4, "use_dynamic_bsz": False,
             "max_token_len_per_gpu": 8192, "truncation": "right",
             # conversations (messages column, optional tools / images columns) instead of prompt / response strings
             "multiturn": {"enable": False, "messages_key": "messages", "tools_key": "tools", "images_key": "images", "max_length": None,
                           "image_min_pixels": None, "image_max_pixels": None},
             "synthetic": {"enable": False, "num_samples": 256, "vocab": 2048, "seed": 0}},
    "model": {"path": None, "preset": None, "override_config": {}, "enable_gradient_checkpointing": False},
    "optim": {"lr": 1e-5, "weight_decay": 0.01, "betas": [0.9, 0.95], "clip_grad": 1.0, "lr_warmup_steps_ratio": 0.1, "lr_scheduler_type": "cosine"},
    "engine": {"strategy": "fsdp", "fsdp_size": -1, "model_dtype": None, "ulysses_sequence_parallel_size": 1, "seed": 0},
    "checkpoint": {"save_contents": ["model", "optimizer", "extra"], "load_contents": ["model", "optimizer", "extra"]},
    "trainer": {"total_epochs": 1, "total_training_steps": None, "project_name": "sft", "experiment_name": "run", "logger": ["console"],
                "default_local_dir": "checkpoints/sft", "save_freq": -1, "test_freq": -1, "resume_mode": "auto", "resume_from_path": None, "max_ckpt_to_keep": None, "default_hdfs_dir": None, "device": "cuda", "nnodes": 1, "n_gpus_per_node": 1},
}


class ConversationWindow(Dataset):
    """A conversation dataset (``verl_b200.utils.dataset.sft_dataset.MultiTurnSFTDataset``: full sequence + per-position loss
    mask) in the prompt / response layout the engine consumes: the first token is the prompt, everything after it the response
    window, and the assistant tokens are the response mask. Image inputs and multimodal positions pass through.
    Reference: ``verl/utils/dataset/multiturn_sft_dataset.py`` feeding ``verl/trainer/sft_trainer.py``."""

    def __init__(self, ds):
        self.ds = ds

    def __len__(self):
        return len(self.ds)

    def __getitem__(self, i):
        it = self.ds[i]
        out = {"input_ids": it["input_ids"], "attention_mask": it["attention_mask"], "position_ids": it["position_ids"],
               "responses": it["input_ids"][1:].clone(), "response_mask": it["loss_mask"][:-1].clone()}      # loss_mask[t]: token t+1 is a target
        if "multi_modal_inputs" in it:
            out["multi_modal_inputs"] = it["multi_modal_inputs"]
        return out


class SFTDataset(Dataset):
    """Rows with ``prompt`` and ``response`` strings (or token-id lists); tokenised when a tokenizer is given."""

    def __init__(self, rows, tokenizer, cfg):
        self.rows, self.tok, self.cfg = rows, tokenizer, cfg
        self.P, self.R = int(cfg.max_prompt_length), int(cfg.max_response_length)

    @classmethod
    def from_files(cls, files, tokenizer, cfg):
        import pandas as pd

        files = [files] if isinstance(files, str) else list(files)
        df = pd.concat([pd.read_parquet(os.path.expanduser(f)) for f in files], ignore_index=True)
        return cls([{"prompt": r[cfg.prompt_key], "response": r[cfg.response_key]} for _, r in df.iterrows()], tokenizer, cfg)

    @classmethod
    def synthetic(cls, cfg):
        g = torch.Generator().manual_seed(int(cfg.synthetic.seed))
        rows = []
        for _ in range(int(cfg.synthetic.num_samples)):
            p = torch.randint(10, int(cfg.synthetic.vocab), (int(torch.randint(4, cfg.max_prompt_length + 1, (1,), generator=g)),), generator=g)
            r = torch.randint(10, int(cfg.synthetic.vocab), (int(torch.randint(4, cfg.max_response_length + 1, (1,), generator=g)),), generator=g)
            rows.append({"prompt": p.tolist(), "response": r.tolist()})
        return cls(rows, None, cfg)

    def _ids(self, x, is_response):
        if isinstance(x, str):
            ids = self.tok(x, add_special_tokens=False)["input_ids"]
            if is_response and self.tok.eos_token_id is not None:
                ids = ids + [self.tok.eos_token_id]
            return ids
        return list(x)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        p = self._ids(self.rows[i]["prompt"], False)[-self.P:]
        r = self._ids(self.rows[i]["response"], True)[: self.R]
        ids = torch.zeros(self.P + self.R, dtype=torch.int64)
        att = torch.zeros(self.P + self.R, dtype=torch.int64)
        ids[self.P - len(p): self.P] = torch.tensor(p)
        att[self.P - len(p): self.P] = 1
        ids[self.P: self.P + len(r)] = torch.tensor(r)
        att[self.P: self.P + len(r)] = 1
        return {"input_ids": ids, "attention_mask": att, "position_ids": VF.compute_position_id_with_mask(att),
                "responses": ids[self.P:].clone(), "response_mask": att[self.P:].clone()}


def build_sft_datasets(config: Config, tokenizer=None, train_dataset=None, val_dataset=None):
    """(train, val) datasets of an SFT run: the ones passed in, else conversations (``data.multiturn.enable``), synthetic rows or
    prompt/response files, as the config says."""
    mc = dict(config.model)
    dc = config.data
    mt = dc.get("multiturn") or {}
    if mt.get("enable", False):
        from verl_b200.models.config import PRESETS, ModelConfig
        from verl_b200.utils.dataset.sft_dataset import MultiTurnSFTDataset

        vis = None
        if mc.get("preset"):
            vis = PRESETS[mc["preset"]].vision
        elif mc.get("path") and os.path.exists(os.path.join(os.path.expanduser(str(mc["path"])), "config.json")):
            vis = ModelConfig.from_pretrained(os.path.expanduser(str(mc["path"]))).vision

        def conversations(files):
            return ConversationWindow(MultiTurnSFTDataset(files, tokenizer, max_length=int(mt.get("max_length") or int(dc.max_prompt_length) + int(dc.max_response_length)),
                                                          messages_key=mt.get("messages_key", "messages"), tools_key=mt.get("tools_key", "tools"),
                                                          truncation=dc.get("truncation", "right"), vision=vis, images_key=mt.get("images_key", "images"),
                                                          image_min_pixels=mt.get("image_min_pixels"), image_max_pixels=mt.get("image_max_pixels")))

        if train_dataset is None:
            train_dataset = conversations(dc.train_files)
        if val_dataset is None and dc.get("val_files"):
            val_dataset = conversations(dc.val_files)
    if train_dataset is None:
        train_dataset = SFTDataset.synthetic(dc) if dc.synthetic.enable else SFTDataset.from_files(dc.train_files, tokenizer, dc)
    if val_dataset is None and dc.get("val_files"):
        val_dataset = SFTDataset.from_files(dc.val_files, tokenizer, dc)
    return train_dataset, val_dataset


class SFTTrainer:
    def __init__(self, config: Config, tokenizer=None, train_dataset=None, val_dataset=None):
        self.config = config
        ensure_process_group()
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        mc = dict(config.model)
        self.engine = EngineRegistry.new("language_model", config.engine.strategy, model_config=Config(mc), engine_config=config.engine,
                                         optimizer_config=config.optim, checkpoint_config=config.checkpoint)
        dc = config.data
        train_dataset, val_dataset = build_sft_datasets(config, tokenizer, train_dataset, val_dataset)
        self.train_dataset, self.val_dataset = train_dataset, val_dataset
        dp, dpr = 1, 0
        per_rank = int(dc.train_batch_size)
        self._dp_from_engine = True
        self.sampler = None
        self.per_rank_bs = per_rank
        steps_per_epoch = max(1, len(train_dataset) // int(dc.train_batch_size))
        total = config.trainer.get("total_training_steps") or steps_per_epoch * int(config.trainer.total_epochs)
        self.total_steps = int(total)
        config.optim["total_training_steps"] = self.total_steps
        self.engine.initialize()
        dp, dpr = self.engine.get_data_parallel_size(), self.engine.get_data_parallel_rank()
        assert int(dc.train_batch_size) % dp == 0
        self.per_rank_bs = int(dc.train_batch_size) // dp
        self.sampler = DistributedSampler(train_dataset, num_replicas=dp, rank=dpr, shuffle=True, seed=0, drop_last=True)
        self.loader = DataLoader(train_dataset, batch_size=self.per_rank_bs, sampler=self.sampler, collate_fn=collate_fn, drop_last=True)
        self.global_step = 0

    def _meta(self):
        dc = self.config.data
        m = {"temperature": 1.0, "calculate_entropy": False, "use_dynamic_bsz": bool(dc.use_dynamic_bsz)}
        if dc.use_dynamic_bsz:
            m["max_token_len_per_gpu"] = int(dc.max_token_len_per_gpu)
        else:
            m["micro_batch_size_per_gpu"] = int(dc.micro_batch_size_per_gpu)
        return m

    def _loss(self, model_output, data, dp_group=None):
        d = dict(data)
        d["loss_mask"] = d["response_mask"]
        return sft_loss(None, model_output, d)

    def train_step(self, batch: dict) -> dict:
        data = DataProto.from_single_dict(batch)
        data.meta_info = self._meta()
        t0 = time.perf_counter()
        with self.engine.train_mode():
            out = self.engine.train_batch(data, self._loss)
            lr = self.engine.lr_scheduler_step()
        m = {k: (v.aggregate() if hasattr(v, "aggregate") else v) for k, v in out["metrics"].items()}
        m = {("train/loss" if k == "sft/loss" else f"train/{k}"): v for k, v in m.items()}
        m["train/lr"] = lr
        m["train/time_s"] = time.perf_counter() - t0
        return m

    @torch.no_grad()
    def validate(self) -> dict:
        if self.val_dataset is None:
            return {}
        loader = DataLoader(self.val_dataset, batch_size=self.per_rank_bs, collate_fn=collate_fn)
        tot, cnt = 0.0, 0.0
        for batch in loader:
            data = DataProto.from_single_dict(batch)
            data.meta_info = self._meta()
            with self.engine.eval_mode():
                mo = self.engine.infer_batch(data)["model_output"]
            mask = data.batch["response_mask"].to(mo["log_probs"].device).float()
            tot += float(-(mo["log_probs"] * mask).sum())
            cnt += float(mask.sum())
        t = torch.tensor([tot, cnt], dtype=torch.float64)
        if dist.is_initialized():
            t = t.to("cuda" if torch.cuda.is_available() else "cpu")
            dist.all_reduce(t)
        return {"val/loss": float(t[0] / t[1].clamp(min=1))}

    def fit(self):
        cfg = self.config.trainer
        logger = Tracking(cfg.project_name, cfg.experiment_name, cfg.logger) if self.rank == 0 else None
        from verl_b200.utils.checkpoint.checkpoint_handler import CheckpointHandler, SkipFirst

        handler = CheckpointHandler(self.engine, default_local_dir=cfg.default_local_dir, max_ckpt_to_keep=cfg.get("max_ckpt_to_keep"),
                                    default_hdfs_dir=cfg.get("default_hdfs_dir"), resume_mode=cfg.get("resume_mode", "auto"),
                                    resume_from_path=cfg.get("resume_from_path"), rank=self.rank)
        self.global_step, pos = handler.load_checkpoint()
        steps_per_epoch = max(1, len(self.loader))
        # a checkpoint without a data position (an older one) continues from where its step count says it was
        pos = pos or {"epoch": self.global_step // steps_per_epoch, "batches": self.global_step % steps_per_epoch}
        skipper = SkipFirst(self.sampler)
        loader = DataLoader(self.train_dataset, batch_size=self.per_rank_bs, sampler=skipper, collate_fn=self.loader.collate_fn, drop_last=True)
        for epoch in range(int(pos["epoch"]), int(cfg.total_epochs) + 1):
            skipper.set_epoch(epoch)
            done = int(pos["batches"]) if epoch == int(pos["epoch"]) else 0
            skipper.skip_next(done * self.per_rank_bs)
            for batch in loader:
                if self.global_step >= self.total_steps:
                    return
                self.global_step += 1
                done += 1
                m = self.train_step(batch)
                if int(cfg.get("test_freq", -1)) > 0 and self.global_step % int(cfg.test_freq) == 0:
                    m.update(self.validate())
                if int(cfg.get("save_freq", -1)) > 0 and (self.global_step % int(cfg.save_freq) == 0 or self.global_step == self.total_steps):
                    handler.save_checkpoint(self.global_step, {"epoch": epoch, "batches": done})
                if logger:
                    logger.log(m, self.global_step)


def main(argv=None):
    import copy

    import yaml

    argv = list(sys.argv[1:] if argv is None else argv)
    data = copy.deepcopy(DEFAULT_CONFIG)
    files = [a for a in argv if a.endswith(".yaml") and "=" not in a]
    for f in files:
        from verl_b200.utils.config import _merge

        _merge(data, yaml.safe_load(open(f)) or {})
    apply_overrides(data, [a for a in argv if a not in files])
    resolve_interpolations(data)
    cfg = Config(data)
    tok = None
    if cfg.model.get("path") and os.path.isdir(os.path.expanduser(cfg.model.path)):
        from verl_b200.trainer.main_ppo import _load_tokenizer

        tok = _load_tokenizer(cfg.model.path)
    elif (cfg.data.get("multiturn") or {}).get("enable", False):
        from verl_b200.utils.tokenizer import ByteChatTokenizer      # preset models without tokenizer files: byte-level chat tokenizer

        tok = ByteChatTokenizer()
    SFTTrainer(cfg, tokenizer=tok).fit()


if __name__ == "__main__":
    main()
