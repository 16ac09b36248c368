"""Curriculum / custom samplers for the RL dataloader (reference: ``verl/experimental/dataset/sampler.py`` —
``AbstractSampler`` / ``AbstractCurriculumSampler`` with an ``update(batch)`` hook called after every step)."""

from __future__ import annotations

from abc import abstractmethod
from typing import Iterator, Optional

import torch
from torch.utils.data import Sampler

__all__ = ["AbstractSampler", "AbstractCurriculumSampler", "DifficultyCurriculumSampler"]


class AbstractSampler(Sampler[int]):
    def __init__(self, data_source, data_config=None):
        self.data_source, self.data_config = data_source, data_config

    def __len__(self):
        return len(self.data_source)


class AbstractCurriculumSampler(AbstractSampler):
    @abstractmethod
    def update(self, batch) -> None:
        """Called with the trained batch (scores included) so the sampler can re-weight what comes next."""


class DifficultyCurriculumSampler(AbstractCurriculumSampler):
    """Keeps a running accuracy per sample index and prefers samples whose accuracy is closest to ``target`` (neither
    solved nor hopeless), mixing in ``explore`` fraction of uniformly random picks."""

    def __init__(self, data_source, data_config=None, target: float = 0.5, explore: float = 0.2, seed: int = 0):
        super().__init__(data_source, data_config)
        self.acc = torch.full((len(data_source),), float("nan"))
        self.target, self.explore = target, explore
        self.gen = torch.Generator().manual_seed(seed)

    def update(self, batch) -> None:
        idx = batch.non_tensor_batch.get("index")
        if idx is None or "token_level_scores" not in batch.batch.keys():
            return
        s = batch.batch["token_level_scores"].sum(-1).float()
        for i, v in zip(idx.tolist(), s.tolist()):
            i = int(i)
            self.acc[i] = v if torch.isnan(self.acc[i]) else 0.8 * float(self.acc[i]) + 0.2 * v

    def __iter__(self) -> Iterator[int]:
        n = len(self.data_source)
        prio = -(torch.nan_to_num(self.acc, nan=self.target) - self.target).abs() + 1e-3 * torch.rand(n, generator=self.gen)
        order = torch.argsort(prio, descending=True).tolist()
        rand = torch.randperm(n, generator=self.gen).tolist()
        for k in range(n):
            yield rand[k] if float(torch.rand(1, generator=self.gen)) < self.explore else order[k]
