"""Variable-resolution / variable-length video batching, and two further index samplers.

* ``VideoBuckets`` -- a bucket is (resolution name, frame count, aspect ratio).  A clip goes to the largest resolution it
  is not much smaller than (80 % of the pixel budget), then to the longest frame count it exceeds, each step passed with
  a configured probability so that long / large buckets can be thinned; every bucket has its own batch size
  (mindspeed_mm/data/data_utils/bucket.py:10-131).  Config: ``{"480p": {1: (0.5, 64), 33: ((1.0, 0.5), 8)}, ...}`` =
  resolution -> frames -> (keep probability or (keep, try-this-length probability), batch size).
* ``VariableVideoBatchSampler`` -- every micro-batch comes from one bucket, the order in which buckets are visited is
  shuffled, ranks take consecutive visits, and the stream can restart after ``consumed`` micro-batches -- also with
  another number of ranks (mindspeed_mm/data/dataloader/sampler.py:690-929).  Yields ``[(index, t, h, w), ...]``.
* ``PaddedDistributedSampler`` -- rank-strided indices, padded (not truncated) so that no sample is dropped, resumable
  inside an epoch (the auto-encoder sampler, sampler.py:931-981).
* ``GroupedLengthSampler`` -- samples carry a task type and a length; inside a task they are sorted by length and
  re-shuffled in windows of 500 global batches, a global batch (and the micro-batches of one accumulation window) holds
  one task only (the Lumina sampler, sampler.py:983-1110).
"""
from __future__ import annotations

import math
from collections import OrderedDict, defaultdict
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Sampler

# pixel budget per named resolution
RESOLUTIONS: Dict[str, int] = {"144p": 256 * 144, "240p": 426 * 240, "256": 256 * 256, "360p": 640 * 360, "480p": 854 * 480,
                               "512": 512 * 512, "720p": 1280 * 720, "1024": 1024 * 1024, "1080p": 1920 * 1080,
                               "2048": 2048 * 2048}
ASPECTS: Tuple[float, ...] = (0.375, 0.43, 0.48, 0.5, 0.53, 0.5625, 0.6, 0.67, 0.75, 0.82, 1.0, 1.21, 1.33, 1.5, 1.67,
                              1.78, 2.0, 2.09, 2.4, 2.67)          # height / width


def aspect_table(pixels: int, multiple: int = 16, aspects: Sequence[float] = ASPECTS) -> "OrderedDict[str, Tuple[int, int]]":
    """Aspect ratio (as a string, height / width) -> (H, W) with about ``pixels`` pixels, both multiples of ``multiple``."""
    out: "OrderedDict[str, Tuple[int, int]]" = OrderedDict()
    for a in aspects:
        h = max(multiple, int(round(math.sqrt(pixels * a) / multiple)) * multiple)
        w = max(multiple, int(round(math.sqrt(pixels / a) / multiple)) * multiple)
        out[f"{a:.2f}"] = (h, w)
    return out


def closest_aspect(h: int, w: int, table: Dict[str, Tuple[int, int]]) -> str:
    r = h / w
    return min(table, key=lambda k: abs(float(k) - r))


class VideoBuckets:
    def __init__(self, config: Dict[str, Dict[int, Sequence]], resolutions: Optional[Dict[str, int]] = None, multiple: int = 16):
        res = dict(RESOLUTIONS, **(resolutions or {}))
        unknown = [k for k in config if k not in res]
        if unknown:
            raise ValueError(f"unknown resolution names {unknown}")
        self.pixels = {k: res[k] for k in config}
        self.tables = {k: aspect_table(res[k], multiple) for k in config}
        # largest resolution first, longest clip first
        self.names = sorted(config, key=lambda k: res[k], reverse=True)
        self.prob: Dict[str, "OrderedDict[int, object]"] = {}
        self.bs: Dict[str, Dict[int, int]] = {}
        self.order: Dict[Tuple[str, int], int] = {}
        for k in self.names:
            frames = sorted((int(t) for t in config[k]), reverse=True)
            get = lambda t, k=k: config[k][t] if t in config[k] else config[k][str(t)]       # noqa: E731
            self.prob[k] = OrderedDict((t, get(t)[0]) for t in frames)
            self.bs[k] = {t: int(get(t)[1]) for t in frames}
            for t in frames:
                self.order[(k, t)] = len(self.order)
        self.num_buckets = sum(len(self.tables[k]) * len(self.prob[k]) for k in self.names)

    def bucket_of(self, T: int, H: int, W: int, seed: int = 0, frame_interval: int = 1) -> Optional[Tuple[str, int, str]]:
        """(resolution, frames, aspect) or None when the clip fits no bucket or lost every draw.  The draws depend on
        (seed, bucket) only, so every rank computes the same assignment."""
        pixels = H * W
        for name in self.names:
            if pixels < 0.8 * self.pixels[name]:
                continue
            probs = self.prob[name]
            chosen, p = None, None
            if T == 1:
                if 1 not in probs:
                    continue
                p = probs[1]
                p = p[0] if isinstance(p, (tuple, list)) else p
                if np.random.default_rng(seed + self.order[(name, 1)]).random() < p:
                    return name, 1, closest_aspect(H, W, self.tables[name])
                continue
            rng = None
            for t, p in probs.items():
                rng = np.random.default_rng(seed + self.order[(name, t)])
                if isinstance(p, (tuple, list)) and rng.random() > p[1]:
                    continue
                if t != 1 and T > t * frame_interval:
                    chosen = t
                    break
            if chosen is None:
                continue
            keep = p[0] if isinstance(p, (tuple, list)) else p
            if keep >= 1 or rng.random() < keep:
                return name, chosen, closest_aspect(H, W, self.tables[name])
        return None

    def thw(self, bucket: Tuple[str, int, str]) -> Tuple[int, int, int]:
        h, w = self.tables[bucket[0]][bucket[2]]
        return bucket[1], h, w

    def batch_size(self, bucket: Tuple[str, int, str]) -> int:
        return self.bs[bucket[0]][bucket[1]]


class VariableVideoBatchSampler(Sampler):
    """``meta[i] = (num_frames, height, width)``.  One iteration = one epoch; ``consumed`` counts micro-batches handed out
    over all ranks and is what ``state_dict`` stores."""

    def __init__(self, meta: Sequence[Tuple[int, int, int]], buckets: VideoBuckets, dp_rank: int = 0, dp_world: int = 1,
                 shuffle: bool = True, seed: int = 0, drop_last: bool = False, frame_interval: int = 1, consumed: int = 0):
        self.meta, self.buckets = list(meta), buckets
        self.dp_rank, self.dp_world = dp_rank, dp_world
        self.shuffle, self.seed, self.drop_last, self.frame_interval = shuffle, seed, drop_last, frame_interval
        self.epoch, self.consumed = 0, consumed

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "consumed": self.consumed, "seed": self.seed}

    def load_state_dict(self, s: dict):
        self.epoch, self.consumed, self.seed = s["epoch"], s["consumed"], s.get("seed", self.seed)

    def group(self) -> "OrderedDict[Tuple[str, int, str], List[int]]":
        groups: "OrderedDict[Tuple[str, int, str], List[int]]" = OrderedDict()
        for i, (t, h, w) in enumerate(self.meta):
            b = self.buckets.bucket_of(t, h, w, self.seed + self.epoch + i * self.buckets.num_buckets, self.frame_interval)
            if b is not None:
                groups.setdefault(b, []).append(i)
        return OrderedDict(sorted(groups.items(), key=lambda kv: (self.buckets.order[(kv[0][0], kv[0][1])], kv[0][2])))

    def _plan(self):
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        groups = self.group()
        visits: List[Tuple[str, int, str]] = []
        for b, idx in groups.items():
            bs = self.buckets.batch_size(b)
            rem = len(idx) % bs
            if rem:
                idx = idx[:-rem] if self.drop_last else idx + (idx * bs)[: bs - rem]
            if self.shuffle:
                idx = [idx[j] for j in torch.randperm(len(idx), generator=g).tolist()]
            groups[b] = idx
            visits += [b] * (len(idx) // bs)
        if self.shuffle:
            visits = [visits[j] for j in torch.randperm(len(visits), generator=g).tolist()]
        rem = len(visits) % self.dp_world
        if rem:
            visits = visits[: len(visits) - rem] if self.drop_last else visits + visits[: self.dp_world - rem]
        return groups, visits

    def __len__(self) -> int:
        return len(self._plan()[1]) // self.dp_world

    def __iter__(self) -> Iterator[List[Tuple[int, int, int, int]]]:
        groups, visits = self._plan()
        iters = len(visits) // self.dp_world
        if iters == 0:
            return
        start = (self.consumed // self.dp_world) % iters
        self.consumed = start * self.dp_world
        used: Dict[Tuple[str, int, str], int] = defaultdict(int)
        for b in visits[: self.consumed]:
            used[b] += self.buckets.batch_size(b)
        for it in range(start, iters):
            mine = None
            for r, b in enumerate(visits[it * self.dp_world: (it + 1) * self.dp_world]):
                bs = self.buckets.batch_size(b)
                if r == self.dp_rank:
                    idx = groups[b]
                    lo = used[b] % len(idx)
                    take = (idx + idx)[lo: lo + bs]
                    mine = [(i, *self.buckets.thw(b)) for i in take]
                used[b] += bs
            self.consumed += self.dp_world
            yield mine
        self.epoch += 1
        self.consumed = 0


class PaddedDistributedSampler(Sampler):
    def __init__(self, n: int, dp_rank: int = 0, dp_world: int = 1, shuffle: bool = True, seed: int = 0, drop_last: bool = False):
        self.n, self.dp_rank, self.dp_world = n, dp_rank, dp_world
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.epoch, self.position = 0, 0
        self.per_rank = n // dp_world if drop_last else math.ceil(n / dp_world)

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "position": self.position}

    def load_state_dict(self, s: dict):
        self.epoch, self.position = s["epoch"], s["position"]

    def __len__(self):
        return self.per_rank

    def __iter__(self):
        order = torch.randperm(self.n, generator=torch.Generator().manual_seed(self.seed + self.epoch)).tolist() \
            if self.shuffle else list(range(self.n))
        total = self.per_rank * self.dp_world
        if len(order) < total:
            order = (order * math.ceil(total / max(len(order), 1)))[:total]
        own = order[:total][self.dp_rank::self.dp_world]
        while self.position < len(own):
            i = own[self.position]
            self.position += 1
            yield i
        self.position = 0
        self.epoch += 1


class GroupedLengthSampler(Sampler):
    """``kinds[i]`` is the task of sample i, ``lengths[i]`` its token count.  Every global batch of
    ``batch_size * dp_world`` samples -- and, unless ``mix_tasks_in_accumulation``, every window of ``acc_grad`` global
    batches -- comes from one task; inside a task neighbours have similar lengths."""

    def __init__(self, kinds: Sequence, lengths: Sequence[int], batch_size: int, dp_rank: int = 0, dp_world: int = 1,
                 acc_grad: int = 1, shuffle: bool = True, seed: int = 0, length_clustering: bool = True,
                 mix_tasks_in_accumulation: bool = False, window: int = 500):
        self.kinds, self.lengths = list(kinds), list(lengths)
        self.bs, self.dp_rank, self.dp_world, self.acc = batch_size, dp_rank, dp_world, acc_grad
        self.shuffle, self.seed, self.cluster, self.mix, self.window = shuffle, seed, length_clustering, mix_tasks_in_accumulation, window
        self.epoch = 0
        unit = batch_size * dp_world * acc_grad
        count = defaultdict(int)
        for k in self.kinds:
            count[k] += 1
        self.total = sum(v // unit * unit for v in count.values())

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __len__(self):
        return self.total // self.dp_world

    def __iter__(self):
        gbs = self.bs * self.dp_world
        unit = gbs * self.acc
        rng = np.random.default_rng(self.seed + self.epoch)
        by_kind: Dict[object, List[int]] = OrderedDict()
        for i, k in enumerate(self.kinds):
            by_kind.setdefault(k, []).append(i)
        batches: List[List[int]] = []
        for k, idx in by_kind.items():
            if self.shuffle:
                rng.shuffle(idx)
            idx = idx[: len(idx) // unit * unit]
            if self.shuffle and self.cluster:
                idx.sort(key=lambda i: self.lengths[i])
                out: List[int] = []
                for s in range(0, len(idx), gbs * self.window):
                    part = idx[s: s + gbs * self.window]
                    rng.shuffle(part)
                    out += part
                idx = out
            chunks = [idx[s: s + gbs] for s in range(0, len(idx), gbs)]
            if self.shuffle and not self.mix:
                rng.shuffle(chunks)
                chunks = [sum(chunks[s: s + self.acc], []) for s in range(0, len(chunks), self.acc)]
            batches += chunks
        if self.shuffle:
            rng.shuffle(batches)
        flat = [i for b in batches for i in b]
        own: List[int] = []
        for s in range(self.dp_rank * self.bs, len(flat), gbs):
            own += flat[s: s + self.bs]
        self.epoch += 1
        return iter(own)
