"""Supervised fine-tuning driven by one controller process.

The torchrun trainer (`verl_b200.trainer.sft_trainer`) runs the data loader on every rank.  Here the data lives on the driver only: it
loads a global batch, orders it so that the data-parallel ranks get similar token counts, and hands it to a worker group whose dispatch
cuts it along the engines' data-parallel axis; the workers (one per GPU, started and supervised by the process worker group) hold the
engine.  Checkpoints go through `CheckpointHandler` in controller mode, so a restarted driver resumes at the same step and the same
position in the data.

    python -m verl_b200.trainer.sft_trainer_controller trainer.n_gpus_per_node=8 model.path=… data.train_files=…

Reference: ``verl/trainer/sft_trainer_ray.py:49-393`` (driver-side ``SFTTrainer`` over a ``TrainingWorker`` group with a
``CheckpointHandler`` in ``OrchestrationMode.RAY``).
"""
from __future__ import annotations

import copy
import sys
import time

import torch
from torch.utils.data import DataLoader, RandomSampler

from verl_b200.protocol import DataProto, collate_fn
from verl_b200.single_controller.base import ClassWithInitArgs, Dispatch, ResourcePool
from verl_b200.single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn, register
from verl_b200.trainer.sft_trainer import DEFAULT_CONFIG, build_sft_datasets
from verl_b200.utils.checkpoint.checkpoint_handler import CheckpointHandler, OrchestrationMode, SkipFirst
from verl_b200.utils.config import Config, apply_overrides, resolve_interpolations
from verl_b200.utils.seqlen_balancing import get_seqlen_balanced_partitions
from verl_b200.utils.tracking import Tracking
from verl_b200.workers.engine_workers import TrainingWorker
from verl_b200.workers.utils.losses import sft_loss

MESH = "sft"


def _masked_nll(model_output, data, dp_group=None):
    d = dict(data)
    d["loss_mask"] = d["response_mask"]
    return sft_loss(None, model_output, d)


class SFTWorker(TrainingWorker):
    """One engine; every call takes this rank's slice of the driver's batch."""

    def __init__(self, config: dict):
        cfg = Config(copy.deepcopy(config))
        super().__init__(Config({"model_type": "language_model", "backend": cfg.engine.strategy, "model": dict(cfg.model), "engine": dict(cfg.engine),
                                 "optim": dict(cfg.optim), "checkpoint": dict(cfg.checkpoint)}), role=MESH)
        self.sft_config = cfg

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        self.reset()
        self.set_loss_fn(_masked_nll)
        return self.engine.get_data_parallel_size()

    def _meta(self) -> dict:
        dc = self.sft_config.data
        m = {"temperature": 1.0, "calculate_entropy": False, "use_dynamic_bsz": bool(dc.use_dynamic_bsz)}
        if dc.use_dynamic_bsz:
            m["max_token_len_per_gpu"] = int(dc.max_token_len_per_gpu)
        else:
            m["micro_batch_size_per_gpu"] = int(dc.micro_batch_size_per_gpu)
        return m

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn(MESH))
    def train_step(self, data: DataProto) -> DataProto:
        data.meta_info = {**self._meta(), **data.meta_info}
        return DataProto(batch=None, non_tensor_batch={}, meta_info={"metrics": self.train_mini_batch(data)})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn(MESH))
    def eval_step(self, data: DataProto) -> DataProto:
        data.meta_info = {**self._meta(), **data.meta_info}
        with torch.no_grad():
            mo = self.infer_batch(data, prefix="")["model_output"]
        mask = data.batch["response_mask"].to(mo["log_probs"].device).float()
        return DataProto.from_dict(tensors={"nll": -(mo["log_probs"] * mask).sum().reshape(1).cpu().double(), "tokens": mask.sum().reshape(1).cpu().double()})


def _balanced(batch: dict, dp: int) -> dict:
    """Reorders the rows so that the ``dp`` equal contiguous chunks the dispatch cuts carry similar token counts."""
    n = batch["attention_mask"].shape[0]
    if dp <= 1 or n % dp:
        return batch
    parts = get_seqlen_balanced_partitions(batch["attention_mask"].sum(-1).tolist(), dp, equal_size=True)
    order = torch.tensor([i for p in parts for i in p])
    return {k: (v[order] if isinstance(v, torch.Tensor) else v[order.numpy()]) for k, v in batch.items()}


class ControllerSFTTrainer:
    def __init__(self, config: Config, tokenizer=None, train_dataset=None, val_dataset=None):
        from verl_b200.single_controller.process import ProcessWorkerGroup

        self.config = config
        tc, dc = config.trainer, config.data
        self.train_dataset, self.val_dataset = build_sft_datasets(config, tokenizer, train_dataset, val_dataset)
        self.batch_size = int(dc.train_batch_size)
        self.sampler = SkipFirst(_EpochShuffle(self.train_dataset, seed=int(dc.get("seed", 0) or 0)))
        self.loader = DataLoader(self.train_dataset, batch_size=self.batch_size, sampler=self.sampler, collate_fn=collate_fn, drop_last=True)
        steps_per_epoch = max(1, len(self.train_dataset) // self.batch_size)
        self.total_steps = int(tc.get("total_training_steps") or steps_per_epoch * int(tc.total_epochs))
        config.optim["total_training_steps"] = self.total_steps
        pool = ResourcePool([int(tc.get("n_gpus_per_node", 1))] * int(tc.get("nnodes", 1)))
        self.wg = ProcessWorkerGroup(pool, ClassWithInitArgs(SFTWorker, config=config.to_dict() if hasattr(config, "to_dict") else dict(config)),
                                     name_prefix="sft", use_gpu=tc.get("device", "cuda") == "cuda")
        self.dp = int(self.wg.init_model()[0])
        assert self.batch_size % self.dp == 0, f"data.train_batch_size={self.batch_size} must divide over {self.dp} data-parallel ranks"
        self.handler = CheckpointHandler(self.wg, default_local_dir=tc.default_local_dir, max_ckpt_to_keep=tc.get("max_ckpt_to_keep"),
                                         default_hdfs_dir=tc.get("default_hdfs_dir"), resume_mode=tc.get("resume_mode", "auto"),
                                         resume_from_path=tc.get("resume_from_path"), mode=OrchestrationMode.CONTROLLER)
        self.global_step = 0

    def validate(self) -> dict:
        if self.val_dataset is None:
            return {}
        nll = tok = 0.0
        for batch in DataLoader(self.val_dataset, batch_size=self.batch_size, collate_fn=collate_fn, drop_last=True):
            out = self.wg.eval_step(DataProto.from_single_dict(batch))
            nll += float(out.batch["nll"].sum())
            tok += float(out.batch["tokens"].sum())
        return {"val/loss": nll / max(tok, 1.0)}

    def fit(self):
        from verl_b200.utils.metric import reduce_metrics

        tc = self.config.trainer
        logger = Tracking(tc.project_name, tc.experiment_name, tc.logger)
        self.global_step, pos = self.handler.load_checkpoint()
        steps_per_epoch = max(1, len(self.loader))
        pos = pos or {"epoch": self.global_step // steps_per_epoch, "batches": self.global_step % steps_per_epoch}
        try:
            for epoch in range(int(pos["epoch"]), int(tc.total_epochs) + 1):
                self.sampler.set_epoch(epoch)
                done = int(pos["batches"]) if epoch == int(pos["epoch"]) else 0
                self.sampler.skip_next(done * self.batch_size)
                for batch in self.loader:
                    if self.global_step >= self.total_steps:
                        return
                    self.global_step += 1
                    done += 1
                    t0 = time.perf_counter()
                    out = self.wg.train_step(DataProto.from_single_dict(_balanced(batch, self.dp)))
                    m = reduce_metrics(out.meta_info["metrics"])
                    m = {("train/loss" if k == "sft/loss" else f"train/{k}"): v for k, v in m.items()}
                    m["train/time_s"] = time.perf_counter() - t0
                    if int(tc.get("test_freq", -1)) > 0 and self.global_step % int(tc.test_freq) == 0:
                        m.update(self.validate())
                    if int(tc.get("save_freq", -1)) > 0 and (self.global_step % int(tc.save_freq) == 0 or self.global_step == self.total_steps):
                        self.handler.save_checkpoint(self.global_step, {"epoch": epoch, "batches": done})
                    logger.log(m, self.global_step)
        finally:
            self.wg.shutdown()


class _EpochShuffle(RandomSampler):
    """A permutation of the dataset that depends on (seed, epoch) only, so a restarted driver draws the same order."""

    def __init__(self, dataset, seed: int = 0):
        super().__init__(dataset)
        self.seed, self.epoch = seed, 0

    def set_epoch(self, epoch: int):
        self.epoch = int(epoch)

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + self.epoch)
        return iter(torch.randperm(len(self.data_source), generator=g).tolist())


def main(argv=None):
    import os

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
        from verl_b200.utils.tokenizer import ByteChatTokenizer

        tok = ByteChatTokenizer()
    ControllerSFTTrainer(cfg, tokenizer=tok).fit()


if __name__ == "__main__":
    main()
