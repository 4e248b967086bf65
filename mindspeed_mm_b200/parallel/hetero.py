"""Per-module parallel plans and per-iteration DP x CP selection.

* ``HeteroPlan`` - different (tp, cp, dp) for the vision tower, the audio tower and the LLM.  The reference
  swaps Megatron's ``mpu`` globals around each sub-module (mindspeed_mm/utils/hetero_parallel.py:22-315); here a
  plan is just a mapping sub-module -> ParallelState-like view, and ``redistribute`` moves the activations between
  the layouts of two neighbouring sub-modules (all-gather over the extra ranks or split among them).
* ``shard_images`` / ``gather_image_rows`` - the plan the Megatron-style backend runs with ``--hetero-parallel``: the
  vision tower is NOT tensor parallel, so instead of every tensor-parallel rank encoding the same images (the
  replicated default), the images of a micro-batch are dealt over the tensor-parallel ranks (longest first onto the
  lightest rank), each rank encodes its share and the merged embeddings are all-gathered back into image order, where
  the tensor-parallel decoder takes over.  Vision parameters then see different data per rank: their gradients are
  summed over the group by the sharding engine (``param._tp_sum_group``).
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


def shard_images(grid_thw: torch.Tensor, world: int, rank: int, merge: int = 2):
    """Deal the images of ``grid_thw`` [n, 3] over ``world`` ranks by patch count.  Returns ``(mine, rows, restore)``:
    this rank's image indices (ascending), the merged-token rows every rank will produce, and the permutation that
    puts the rank-major concatenation of all ranks' outputs back into image order.  ``None`` when there are fewer
    images than ranks (every rank then encodes everything, as without the plan)."""
    from ..data.packing import balance_across_ranks
    counts = grid_thw.prod(-1).tolist()
    if len(counts) < world:
        return None
    parts = [sorted(p) for p in balance_across_ranks(counts, world)]
    unit = merge * merge
    tokens = [c // unit for c in counts]
    rows = [sum(tokens[i] for i in p) for p in parts]
    starts = [0]
    for t in tokens:
        starts.append(starts[-1] + t)
    # gathered order: rank 0's images, rank 1's, ...; restore[k] = position in the gathered tensor of original row k
    src = torch.cat([torch.arange(starts[i], starts[i + 1]) for p in parts for i in p])
    restore = torch.empty_like(src)
    restore[src] = torch.arange(src.numel())
    return parts[rank], rows, restore


class _GatherRows(torch.autograd.Function):
    """All-gather of per-rank row blocks of different heights (padded to the tallest for the collective).  The consumer's
    gradient is identical on all ranks of the group (it comes out of a replicated or all-gathered tensor), so the
    backward just hands each rank the rows it contributed."""

    @staticmethod
    def forward(ctx, x, rows, group):
        ctx.rows, ctx.rank = rows, dist.get_rank(group)
        world, top = len(rows), max(rows)
        pad = x.new_zeros(top, *x.shape[1:])
        pad[:x.shape[0]] = x
        out = x.new_empty(world * top, *x.shape[1:])
        dist.all_gather_into_tensor(out, pad, group=group)
        return torch.cat([out[r * top:r * top + rows[r]] for r in range(world)])

    @staticmethod
    def backward(ctx, g):
        lo = sum(ctx.rows[:ctx.rank])
        return g[lo:lo + ctx.rows[ctx.rank]].contiguous(), None, None


def gather_image_rows(x: torch.Tensor, rows: Sequence[int], restore: torch.Tensor, group) -> torch.Tensor:
    """Merged-token rows of this rank's images -> rows of all images, in image order, on every rank of ``group``."""
    return _GatherRows.apply(x, list(rows), group).index_select(0, restore.to(x.device))


def choose_dp_cp(seq_lens: Sequence[int], world: int, max_tokens_per_rank: int, allowed=(1, 2, 4, 8)) -> Dict[str, int]:
    longest = max(seq_lens)
    cp = next((c for c in allowed if c <= world and world % c == 0 and (longest + c - 1) // c <= max_tokens_per_rank), None)
    if cp is None:
        raise ValueError(f"a sequence of {longest} tokens does not fit {max_tokens_per_rank} tokens per rank with cp <= {world}")
    return {"cp": cp, "dp": world // cp}
