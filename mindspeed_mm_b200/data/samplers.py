"""Batch samplers with resumable state.

* ``StatefulDistributedSampler`` - rank-strided sampling that can restart at ``consumed_samples``.
* ``BaseRandomBatchSampler``     - epoch-shuffled batches of the micro-batch size per data-parallel rank
                                   (the default sampler of the recipes: ``sampler_type: BaseRandomBatchSampler``).
* ``LengthGroupedSampler``       - megabatches sorted by length so a batch has little padding.
* ``BucketBatchSampler``         - samples are put in (frames, height, width)-style buckets; every batch
                                   comes from one bucket (variable-resolution video training).
Reference: mindspeed_mm/data/dataloader/sampler.py:284-983, fsdp/data/dataloader/sampler.py:8.
Every sampler is a pure function of (seed, epoch, consumed samples): ``state_dict`` / ``load_state_dict`` make
resume exact, and ``set_epoch`` reshuffles.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Hashable, Iterator, List, Optional, Sequence

import torch
from torch.utils.data import Sampler


class _Resumable(Sampler):
    def __init__(self, n: int, dp_rank: int, dp_world: int, seed: int = 0, shuffle: bool = True, drop_last: bool = True,
                 consumed_samples: int = 0):
        self.n, self.dp_rank, self.dp_world = n, dp_rank, dp_world
        self.seed, self.shuffle, self.drop_last = seed, shuffle, drop_last
        self.epoch, self.consumed = 0, consumed_samples

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "consumed": self.consumed, "seed": self.seed}

    def load_state_dict(self, s):
        self.epoch, self.consumed, self.seed = s["epoch"], s["consumed"], s.get("seed", self.seed)

    def _perm(self) -> List[int]:
        if not self.shuffle:
            return list(range(self.n))
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        return torch.randperm(self.n, generator=g).tolist()


class StatefulDistributedSampler(_Resumable):
    def __iter__(self) -> Iterator[int]:
        order = self._perm()
        total = len(order) // self.dp_world * self.dp_world if self.drop_last else len(order)
        start = self.consumed % max(total, 1)
        for i in range(start + self.dp_rank, total, self.dp_world):
            self.consumed += self.dp_world
            yield order[i]
        self.epoch += 1
        self.consumed = 0

    def __len__(self):
        return self.n // self.dp_world


class BaseRandomBatchSampler(_Resumable):
    """Yields lists of ``micro_batch_size`` indices for this data-parallel rank; runs forever over epochs."""

    def __init__(self, n, micro_batch_size, dp_rank, dp_world, **kw):
        super().__init__(n, dp_rank, dp_world, **kw)
        self.mbs = micro_batch_size
        self.global_mbs = micro_batch_size * dp_world

    def __iter__(self) -> Iterator[List[int]]:
        while True:
            order = self._perm()
            usable = len(order) // self.global_mbs * self.global_mbs if self.drop_last else len(order)
            if usable == 0:
                raise ValueError(f"dataset of {self.n} samples is smaller than one global micro-batch {self.global_mbs}")
            pos = self.consumed % usable if self.consumed else 0
            while pos + self.global_mbs <= usable:
                lo = pos + self.dp_rank * self.mbs
                self.consumed += self.global_mbs
                pos += self.global_mbs
                yield order[lo:lo + self.mbs]
            self.epoch += 1
            self.consumed = 0

    def __len__(self):
        return self.n // self.global_mbs


class LengthGroupedSampler(_Resumable):
    def __init__(self, lengths: Sequence[int], micro_batch_size, dp_rank, dp_world, group_factor: int = 50, **kw):
        super().__init__(len(lengths), dp_rank, dp_world, **kw)
        self.lengths, self.mbs, self.group_factor = list(lengths), micro_batch_size, group_factor

    def __iter__(self):
        order = self._perm()
        gmb = self.mbs * self.dp_world
        mega = gmb * self.group_factor
        batches = []
        for s in range(0, len(order), mega):
            chunk = sorted(order[s:s + mega], key=lambda i: -self.lengths[i])
            batches += [chunk[b:b + gmb] for b in range(0, len(chunk) - gmb + 1, gmb)]
        g = torch.Generator().manual_seed(self.seed + self.epoch + 1)
        for bi in torch.randperm(len(batches), generator=g).tolist():
            b = batches[bi]
            yield b[self.dp_rank * self.mbs:(self.dp_rank + 1) * self.mbs]
        self.epoch += 1

    def __len__(self):
        return self.n // (self.mbs * self.dp_world)


class BucketBatchSampler(_Resumable):
    """``bucket_of(i)`` returns a hashable bucket id (e.g. (frames, h, w)); ``batch_size_of(bucket)`` lets
    large-resolution buckets use smaller batches."""

    def __init__(self, n, bucket_of: Callable[[int], Hashable], batch_size_of: Callable[[Hashable], int], dp_rank,
                 dp_world, **kw):
        super().__init__(n, dp_rank, dp_world, **kw)
        self.bucket_of, self.batch_size_of = bucket_of, batch_size_of

    def __iter__(self):
        buckets: Dict[Hashable, List[int]] = {}
        for i in self._perm():
            buckets.setdefault(self.bucket_of(i), []).append(i)
        batches = []
        for b, idx in sorted(buckets.items(), key=lambda kv: str(kv[0])):
            bs = self.batch_size_of(b) * self.dp_world
            batches += [(b, idx[s:s + bs]) for s in range(0, len(idx) - bs + 1, bs)]
        g = torch.Generator().manual_seed(self.seed + self.epoch + 7)
        for bi in torch.randperm(len(batches), generator=g).tolist():
            b, idx = batches[bi]
            per = len(idx) // self.dp_world
            yield idx[self.dp_rank * per:(self.dp_rank + 1) * per]
        self.epoch += 1


SAMPLERS = {"BaseRandomBatchSampler": BaseRandomBatchSampler, "LengthGroupedSampler": LengthGroupedSampler,
            "BucketBatchSampler": BucketBatchSampler, "StatefulDistributedSampler": StatefulDistributedSampler}


def _late():
    """The bucketed-video, padded and grouped-length samplers live in ``video_buckets.py``; listed here under the names the
    recipes use (``sampler_type``)."""
    from .video_buckets import GroupedLengthSampler, PaddedDistributedSampler, VariableVideoBatchSampler
    SAMPLERS.update({"VariableVideoBatchSampler": VariableVideoBatchSampler, "AESampler": PaddedDistributedSampler,
                     "LuminaMetaLenDistSampler": GroupedLengthSampler})


_late()
