"""A resumable dataloader: iteration position and sampler RNG are part of ``state_dict``.

Stands in for ``torchdata.stateful_dataloader.StatefulDataLoader`` as used by
``verl/trainer/ppo/ray_trainer.py:374-451`` (``data.pt`` in the checkpoint).
"""

from __future__ import annotations

from typing import Callable, Iterator, Optional

import torch
from torch.utils.data import Dataset, Sampler

__all__ = ["StatefulDataLoader", "ShardedRandomSampler", "ShardedSequentialSampler"]


class ShardedSequentialSampler(Sampler):
    def __init__(self, n: int, rank: int = 0, world: int = 1):
        self.n, self.rank, self.world = n, rank, world

    def __iter__(self):
        return iter(range(self.rank, self.n - self.n % self.world, self.world))

    def __len__(self):
        return self.n // self.world

    def set_epoch(self, e: int) -> None:
        pass


class ShardedRandomSampler(Sampler):
    """Seeded permutation per epoch; rank ``r`` of ``world`` takes every ``world``-th index."""

    def __init__(self, n: int, seed: int = 1, rank: int = 0, world: int = 1):
        self.n, self.seed, self.rank, self.world, self.epoch = n, seed, rank, world, 0

    def set_epoch(self, e: int) -> None:
        self.epoch = e

    def __iter__(self):
        g = torch.Generator()
        g.manual_seed(self.seed + self.epoch)
        perm = torch.randperm(self.n, generator=g).tolist()
        usable = self.n - self.n % self.world
        return iter(perm[self.rank:usable:self.world])

    def __len__(self):
        return self.n // self.world


class StatefulDataLoader:
    def __init__(self, dataset: Dataset, batch_size: int = 1, shuffle: bool = False, sampler: Optional[Sampler] = None,
                 collate_fn: Optional[Callable] = None, drop_last: bool = False, num_workers: int = 0, seed: int = 1, **_):
        self.dataset, self.batch_size, self.collate_fn, self.drop_last = dataset, int(batch_size), collate_fn, drop_last
        self.sampler = sampler if sampler is not None else (
            ShardedRandomSampler(len(dataset), seed) if shuffle else ShardedSequentialSampler(len(dataset)))
        self.epoch = 0
        self.batches_yielded = 0
        self._resume_skip = 0

    def __len__(self) -> int:
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def __iter__(self) -> Iterator:
        if hasattr(self.sampler, "set_epoch"):
            self.sampler.set_epoch(self.epoch)
        idx = list(iter(self.sampler))
        skip, self._resume_skip = self._resume_skip, 0
        self.batches_yielded = skip
        for s in range(skip * self.batch_size, len(idx), self.batch_size):
            chunk = idx[s : s + self.batch_size]
            if len(chunk) < self.batch_size and self.drop_last:
                break
            items = [self.dataset[i] for i in chunk]
            self.batches_yielded += 1
            yield self.collate_fn(items) if self.collate_fn is not None else items
        self.epoch += 1
        self.batches_yielded = 0

    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "batches_yielded": self.batches_yielded}

    def load_state_dict(self, st: dict) -> None:
        self.epoch = int(st.get("epoch", 0))
        self._resume_skip = int(st.get("batches_yielded", 0))
        if self._resume_skip >= len(self):
            self.epoch += 1
            self._resume_skip = 0
