"""Per-module parallel plans and per-iteration DP x CP selection.

* ``HeteroPlan`` - different (tp, cp, dp) for the vision tower, the audio tower and the LLM.  The reference
  swaps Megatron's ``mpu`` globals around each sub-module (mindspeed_mm/utils/hetero_parallel.py:22-315); here a
  plan is just a mapping sub-module -> ParallelState-like view, and ``redistribute`` moves the activations between
  the layouts of two neighbouring sub-modules (all-gather over the extra ranks or split among them).
* ``choose_dp_cp`` - dynamic DP / CP: given the sequence lengths of the coming global batch, pick the smallest
  context-parallel degree that fits ``max_tokens_per_rank`` (longer samples get more ranks), the rest is data
  parallel (mindspeed_mm/utils/dpcp_utils.py:63-258).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

import torch
import torch.distributed as dist

from .cp.split import gather_forward_split_backward, split_forward_gather_backward


@dataclass
class ModulePlan:
    tp: int = 1
    cp: int = 1
    pp: int = 1

    def dp(self, world: int) -> int:
        return world // (self.tp * self.cp * self.pp)


class HeteroPlan:
    def __init__(self, world: int, plans: Dict[str, ModulePlan]):
        self.world, self.plans = world, plans
        for name, p in plans.items():
            if world % (p.tp * p.cp * p.pp):
                raise ValueError(f"{name}: tp*cp*pp = {p.tp * p.cp * p.pp} does not divide world {world}")

    def describe(self) -> str:
        return ", ".join(f"{n}: tp{p.tp} cp{p.cp} pp{p.pp} dp{p.dp(self.world)}" for n, p in self.plans.items())


def redistribute(x: torch.Tensor, src: ModulePlan, dst: ModulePlan, group, dim: int = 0):
    """Move a token-major activation from ``src`` layout to ``dst`` layout over ``group`` (the ranks that differ).
    More data-parallel ranks downstream -> split; fewer -> gather."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    s, d = src.tp * src.cp, dst.tp * dst.cp
    if d > s:        # downstream shards the sequence more: every rank keeps its slice
        return split_forward_gather_backward(x, group, dim=dim)
    if d < s:
        return gather_forward_split_backward(x, group, dim=dim)
    return x


def choose_dp_cp(seq_lens: Sequence[int], world: int, max_tokens_per_rank: int, allowed=(1, 2, 4, 8)) -> Dict[str, int]:
    longest = max(seq_lens)
    cp = next((c for c in allowed if c <= world and world % c == 0 and (longest + c - 1) // c <= max_tokens_per_rank), None)
    if cp is None:
        raise ValueError(f"a sequence of {longest} tokens does not fit {max_tokens_per_rank} tokens per rank with cp <= {world}")
    return {"cp": cp, "dp": world // cp}
