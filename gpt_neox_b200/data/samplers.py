"""Index samplers for the training data loaders.

``DistributedBatchSampler`` walks an index sampler, groups the indices into *global* batches and hands every
data-parallel rank its contiguous share of each one, so that all ranks together see exactly the sampler's
order.  ``start_iter`` makes the first pass skip the batches an interrupted run already consumed (counted in
optimizer steps of ``gradient_accumulation_steps`` micro-batches), which is how training resumes mid-epoch.
``RandomSampler`` is a permutation (or with-replacement) sampler whose stream is a pure function of the epoch
number set with ``set_epoch``.  Behavioural counterpart of megatron/data/samplers.py.
"""
from __future__ import annotations

from typing import Iterator, List

import torch
from torch.utils.data import BatchSampler, Sampler


class RandomSampler(Sampler):
    def __init__(self, data_source, replacement: bool = False, num_samples: int | None = None):
        if not isinstance(replacement, bool):
            raise ValueError(f"replacement should be a boolean value, but got replacement={replacement}")
        if num_samples is not None and not replacement:
            raise ValueError("With replacement=False, num_samples should not be specified, since a random "
                             "permute will be performed.")
        self.data_source, self.replacement, self._requested = data_source, replacement, num_samples
        if not isinstance(self.num_samples, int) or self.num_samples <= 0:
            raise ValueError(f"num_samples should be a positive integer value, but got num_samples={self.num_samples}")
        self.epoch = -1

    @property
    def num_samples(self) -> int:
        return self._requested if self._requested is not None else len(self.data_source)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _generator(self) -> torch.Generator:
        g = torch.Generator()
        if self.epoch >= 0:             # before the first set_epoch the stream is left unseeded
            g.manual_seed(self.epoch)
        return g

    def __iter__(self) -> Iterator[int]:
        n, g = len(self.data_source), self._generator()
        order = torch.randint(n, (self.num_samples,), dtype=torch.int64, generator=g) if self.replacement \
            else torch.randperm(n, generator=g)
        return iter(order.tolist())

    def __len__(self) -> int:
        return self.num_samples


class DistributedBatchSampler(BatchSampler):
    def __init__(self, sampler, batch_size: int, drop_last: bool, rank: int = -1, world_size: int = 2,
                 wrap_last: bool = False, gradient_accumulation_steps: int | None = None):
        if rank < 0:
            raise ValueError("DistributedBatchSampler needs the data-parallel rank of this process")
        super().__init__(sampler, batch_size, drop_last)
        self.rank, self.world_size, self.wrap_last = rank, world_size, wrap_last
        # `wrap_around` = how many leading indices of the next pass were already served as the tail of the
        # previous pass's padded last batch (only with wrap_last)
        self.wrap_around = 0
        self.sampler.wrap_around = 0
        self.start_iter = 0
        self.effective_batch_size = batch_size * (gradient_accumulation_steps or 1)

    def _share(self, global_batch: List[int]) -> List[int]:
        lo = self.rank * self.batch_size // self.world_size
        hi = (self.rank + 1) * self.batch_size // self.world_size
        return global_batch[lo:hi]

    def data_iterator(self, indices, wrap_around: bool = False):
        skip = self.wrap_around % self.batch_size
        for n, idx in enumerate(indices):
            if n < skip:
                continue
            if wrap_around:
                self.wrap_around = (self.wrap_around + 1) % self.batch_size
            yield idx

    def __iter__(self):
        pending: List[int] = []
        seen = 0                                        # indices passed so far in this pass
        resume_after = self.start_iter * self.effective_batch_size
        for idx in self.data_iterator(self.sampler, wrap_around=False):
            pending.append(idx)
            if len(pending) < self.batch_size:
                continue
            if seen >= resume_after:
                yield self._share(pending)
                self.start_iter, resume_after = 0, 0     # the skip applies to the first pass only
            seen += self.batch_size
            pending = []
        if pending and not self.drop_last:
            if self.wrap_last:
                self.sampler.wrap_around -= self.batch_size
                self.wrap_around = (self.wrap_around + len(pending)) % self.batch_size
            yield self._share(pending)
        if self.wrap_last:
            self.sampler.wrap_around += self.batch_size
