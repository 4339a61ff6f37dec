"""Deterministic, resumable distributed sampler (reference: ``astrai/dataset/sampler.py:8-84``).

Order = ``randperm(len, seed + epoch)`` padded by wrap-around to a multiple of the world size,
then the rank-strided slice; ``start_iter`` samples are skipped once (resume), and the epoch
advances automatically when an iteration finishes.
"""

from __future__ import annotations

from typing import Iterator, Optional

import torch
from torch.utils.data import Sampler

from ..parallel.setup import get_rank, get_world_size


class ResumableDistributedSampler(Sampler[int]):
    def __init__(self, data_source, start_epoch: int = 0, start_iter: int = 0, seed: int = 42,
                 drop_last: bool = False, shuffle: bool = True, process_group=None,
                 num_replicas: Optional[int] = None, rank: Optional[int] = None):
        self.data_source = data_source
        self.num_replicas = num_replicas if num_replicas is not None else get_world_size()
        self.rank = rank if rank is not None else get_rank()
        self.epoch, self.iter = start_epoch, start_iter
        self.seed, self.shuffle, self.drop_last = seed, shuffle, drop_last
        self._size()

    def _size(self) -> None:
        n = len(self.data_source)
        if self.drop_last and n % self.num_replicas:
            self.num_samples = n // self.num_replicas
        else:
            self.num_samples = (n + self.num_replicas - 1) // self.num_replicas
        self.total_size = self.num_samples * self.num_replicas

    def set_replicas(self, num_replicas: int, rank: int) -> None:
        """Re-partition the data (tensor-parallel ranks all read the same samples: one replica)."""
        self.num_replicas, self.rank = num_replicas, rank
        self._size()

    def _order(self) -> list:
        n = len(self.data_source)
        if self.shuffle:
            gen = torch.Generator()
            gen.manual_seed(self.seed + self.epoch)
            order = torch.randperm(n, generator=gen).tolist()
        else:
            order = list(range(n))
        if self.drop_last:
            order = order[: self.total_size]
        elif order:
            while len(order) < self.total_size:
                order += order[: self.total_size - len(order)]
        return order[self.rank:self.total_size:self.num_replicas]

    def __iter__(self) -> Iterator[int]:
        mine = self._order()
        for idx in mine[self.iter:]:
            self.iter += 1
            yield idx
        self.epoch += 1
        self.iter = 0

    def __len__(self) -> int:
        return max(self.num_samples - self.iter, 0)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch
