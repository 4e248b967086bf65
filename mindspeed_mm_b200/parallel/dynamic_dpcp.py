"""Per-iteration choice of the data-parallel x context-parallel split.

A batch of short sequences wants every rank on its own sample (``dp = W, cp = 1``); one very long sequence needs its
tokens spread over several ranks (``cp > 1``).  ``DynamicDPCP`` builds the process groups of every split ``W = dp x cp``
(``cp`` a power of two up to ``max_cp``) once, then per iteration:

1. ``choose``: the longest sequence of the iteration (max over all ranks) picks the smallest ``cp`` whose share fits
   ``max_tokens_per_rank``;
2. ``switch``: the context-parallel / data-parallel groups of that split become the current ones (also in the
   ``ParallelState`` when one is given, under ``cp`` / ``ulysses`` / ``dp``), after a barrier;
3. ``redistribute``: with ``cp > 1`` the members of a context-parallel group exchange their batches; each member returns
   the list of the group's batches, to be run one after the other with the sequence split over the group.  Samples per
   iteration and the global batch stay what they were: the group does ``cp`` micro-steps on ``cp``-way split sequences
   instead of one step on whole sequences.

Reference: mindspeed_mm/utils/dpcp_utils.py (``initialize_parall_switch_list`` :81, ``modify_parallel`` :115,
``data_aware_parallel_optimize`` :169, the batch broadcast :221-258).  Context-parallel ranks are consecutive (the
``tp-cp-ep-dp-pp`` order of the reference with tp = 1), so a context-parallel group stays inside one NVLink domain.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .hetero import choose_dp_cp


class DynamicDPCP:
    def __init__(self, max_tokens_per_rank: int, max_cp: int = 8, group: Optional[dist.ProcessGroup] = None,
                 parallel_state=None, timeout=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_tokens = max_tokens_per_rank
        self.ps = parallel_state
        self.options: List[int] = []
        self._cp_groups: Dict[int, Optional[dist.ProcessGroup]] = {}
        self._dp_groups: Dict[int, Optional[dist.ProcessGroup]] = {}
        self._cp_ranks: Dict[int, List[int]] = {}
        to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
        cp = 1
        while cp <= min(max_cp, self.world) and self.world % cp == 0:
            self.options.append(cp)
            # every rank creates every group (group creation is collective), and remembers its own
            for start in range(0, self.world, cp):
                ranks = [to_global(r) for r in range(start, start + cp)]
                g = dist.new_group(ranks, timeout=timeout) if cp > 1 else None
                if self.rank in range(start, start + cp):
                    self._cp_groups[cp], self._cp_ranks[cp] = g, ranks
            for off in range(cp):
                ranks = [to_global(r) for r in range(off, self.world, cp)]
                g = dist.new_group(ranks, timeout=timeout) if len(ranks) > 1 else None
                if self.rank % cp == off:
                    self._dp_groups[cp] = g
            cp *= 2
        self.cp = 1

    # -- 1 ---------------------------------------------------------------------------------------------------------
    def choose(self, local_seq_lens: Sequence[int]) -> Tuple[int, int]:
        longest = torch.tensor([max(local_seq_lens) if len(local_seq_lens) else 0], dtype=torch.int64)
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl" else torch.device("cpu")
        longest = longest.to(dev)
        dist.all_reduce(longest, op=dist.ReduceOp.MAX, group=self.group)
        plan = choose_dp_cp([int(longest)], self.world, self.max_tokens, allowed=tuple(self.options))
        return plan["cp"], plan["dp"]

    # -- 2 ---------------------------------------------------------------------------------------------------------
    def switch(self, cp: int) -> None:
        if cp not in self._cp_groups and cp != 1:
            raise ValueError(f"cp={cp} is not one of the prepared splits {self.options}")
        dist.barrier(group=self.group)          # nobody still runs collectives of the previous split
        self.cp = cp
        if self.ps is not None:
            ps = self.ps
            for name in ("cp", "ulysses"):
                ps._groups[name], ps._sizes[name] = self._cp_groups.get(cp), cp
            ps._sizes["ring"] = 1
            ps._groups["dp"], ps._sizes["dp"] = self._dp_groups.get(cp), self.world // cp

    @property
    def cp_group(self) -> Optional[dist.ProcessGroup]:
        return self._cp_groups.get(self.cp)

    @property
    def dp_group(self) -> Optional[dist.ProcessGroup]:
        return self._dp_groups.get(self.cp)

    @property
    def cp_rank(self) -> int:
        return self.rank % self.cp

    # -- 3 ---------------------------------------------------------------------------------------------------------
    def redistribute(self, batch) -> list:
        """-> the batches of this rank's context-parallel group, in rank order (``[batch]`` when ``cp == 1``)."""
        if self.cp == 1:
            return [batch]
        out: list = [None] * self.cp
        dist.all_gather_object(out, _to_cpu(batch), group=self.cp_group)
        dev = _first_device(batch)
        return [_to_device(b, dev) for b in out]

    def step(self, batch, seq_lens: Sequence[int]) -> list:
        """choose + switch + redistribute for one iteration."""
        cp, _ = self.choose(seq_lens)
        if cp != self.cp:
            self.switch(cp)
        return self.redistribute(batch)


def _map(obj, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, dict):
        return {k: _map(v, fn) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_map(v, fn) for v in obj)
    return obj


def _to_cpu(batch):
    return _map(batch, lambda t: t.detach().cpu())


def _to_device(batch, dev):
    return batch if dev is None or dev.type == "cpu" else _map(batch, lambda t: t.to(dev, non_blocking=True))


def _first_device(obj):
    found: list = []
    _map(obj, lambda t: found.append(t.device) or t)
    return found[0] if found else None
