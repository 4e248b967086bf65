"""Dynamic batching: pack variable-length samples into micro-batches of at most ``max_seq_len`` tokens.

A buffer of ``buffer_size`` samples is kept; each micro-batch is filled greedily (longest sample that still
fits first), so padding disappears and every micro-batch is one packed TND stream.  Reference:
mindspeed_mm/data/dataloader/dynamic_batching_dataloader.py:37-159 and batching_strategy.py:16-130.
``balance_across_ranks`` is the host part of data balancing (greedy longest-processing-time assignment of
samples to data-parallel ranks by cost, mindspeed_mm/utils/utils.py:388 ``dist_sort``).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Iterator, List, Sequence, Tuple


def greedy_pack(lengths: Sequence[int], max_seq_len: int) -> List[List[int]]:
    """First-fit-decreasing bins of indices; a sample longer than the budget gets a bin of its own."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: List[Tuple[int, List[int]]] = []
    for i in order:
        for b, (used, idx) in enumerate(bins):
            if used + lengths[i] <= max_seq_len:
                bins[b] = (used + lengths[i], idx + [i])
                break
        else:
            bins.append((lengths[i], [i]))
    return [idx for _, idx in bins]


class DynamicBatcher:
    """Wraps a sample iterator; yields lists of samples whose total length fits the budget."""

    def __init__(self, samples: Iterable[dict], max_seq_len: int, buffer_size: int = 200,
                 length_of: Callable[[dict], int] = lambda s: len(s["input_ids"])):
        self.samples, self.max_seq_len, self.buffer_size, self.length_of = samples, max_seq_len, buffer_size, length_of

    def __iter__(self) -> Iterator[List[dict]]:
        buf: List[dict] = []
        it = iter(self.samples)
        done = False
        while True:
            while not done and len(buf) < self.buffer_size:
                try:
                    buf.append(next(it))
                except StopIteration:
                    done = True
            if not buf:
                return
            buf.sort(key=self.length_of, reverse=True)
            take, used, rest = [], 0, []
            for s in buf:
                n = self.length_of(s)
                if not take or used + n <= self.max_seq_len:
                    take.append(s)
                    used += n
                else:
                    rest.append(s)
            buf = rest
            yield take


def balance_across_ranks(costs: Sequence[float], world: int) -> List[List[int]]:
    """LPT: heaviest item to the currently lightest rank.  Returns per-rank index lists."""
    loads = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(costs)), key=lambda i: -costs[i]):
        r = min(range(world), key=lambda r: loads[r])
        out[r].append(i)
        loads[r] += costs[i]
    return out
