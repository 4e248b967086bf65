"""Online data balancing of vision-encoder work across data-parallel ranks.

Images are unevenly distributed over ranks after packing; the ViT cost of a rank is proportional to its patch
count.  ``balance_images`` computes a global greedy assignment (longest processing time first) from the
all-gathered per-image patch counts, ``EncoderBalance`` moves the patch tensors with an all-to-all before the
ViT and moves the resulting embeddings back afterwards (differentiable in both directions).  Reference:
mindspeed_mm/utils/data_balance/data_balance.py:21-376, ``dist_sort`` and ``EncoderBalanceComm``
(mindspeed_mm/utils/utils.py:388-497).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from ..data.packing import balance_across_ranks


def balance_images(all_counts: Sequence[Sequence[int]]) -> List[List[Tuple[int, int]]]:
    """``all_counts[r]`` = patch counts of rank r's images.  Returns per destination rank a list of (src, index)."""
    items = [(r, i, c) for r, cs in enumerate(all_counts) for i, c in enumerate(cs)]
    parts = balance_across_ranks([c for _, _, c in items], len(all_counts))
    return [[(items[j][0], items[j][1]) for j in sorted(p)] for p in parts]


class _ListAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, in_rows, out_rows, x):
        ctx.group, ctx.in_rows, ctx.out_rows = group, in_rows, out_rows
        out = x.new_empty(sum(out_rows), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_rows, input_split_sizes=in_rows, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty(sum(ctx.in_rows), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_rows, input_split_sizes=ctx.out_rows, group=ctx.group)
        return None, None, None, out


class EncoderBalance:
    def __init__(self, group):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)

    def plan(self, my_counts: List[int], my_grids=None):
        allc: List[List[int]] = [None] * self.world
        dist.all_gather_object(allc, list(my_counts), group=self.group)
        if my_grids is not None:                       # (t, h, w) of every image, so that receivers can index theirs
            self.all_grids = [None] * self.world
            dist.all_gather_object(self.all_grids, [list(map(int, g)) for g in my_grids], group=self.group)
        assign = balance_images(allc)
        self.assign = assign
        # rows I send to each destination, in (dst, my image index) order; rows I receive from each source
        send = [[i for (s, i) in assign[d] if s == self.rank] for d in range(self.world)]
        recv = [[allc[s][i] for (s2, i) in assign[self.rank] if s2 == s] for s in range(self.world)]
        return allc, send, recv

    def dispatch(self, patches: torch.Tensor, my_counts: List[int], my_grids=None):
        """patches: [sum(my_counts), C] -> balanced patches on this rank + the bookkeeping to undo it.  With
        ``my_grids`` the bookkeeping also lists the (t, h, w) of the images this rank now holds, in arrival order."""
        allc, send, recv = self.plan(my_counts, my_grids)
        if any(len(a) == 0 for a in self.assign):      # fewer images than ranks: every rank keeps its own (same decision
            return patches, None                       # everywhere, since the counts were all-gathered)
        starts = [0]
        for c in my_counts:
            starts.append(starts[-1] + c)
        order = [i for d in range(self.world) for i in send[d]]
        idx = torch.cat([torch.arange(starts[i], starts[i + 1]) for i in order]) if order else torch.zeros(0, dtype=torch.long)
        in_rows = [sum(my_counts[i] for i in send[d]) for d in range(self.world)]
        out_rows = [sum(r) for r in recv]
        x = _ListAllToAll.apply(self.group, in_rows, out_rows, patches.index_select(0, idx.to(patches.device)))
        book = dict(idx=idx, in_rows=in_rows, out_rows=out_rows, recv=recv)
        if my_grids is not None:                       # arrival order: by source rank, then by the source's image index
            mine = sorted(self.assign[self.rank])
            book["grids"] = torch.tensor([self.all_grids[s][i] for s, i in mine], dtype=torch.long).view(-1, 3)
        return x, book

    def combine(self, feats: torch.Tensor, book: dict, ratio: int = 1):
        """Inverse movement for per-patch (ratio=1) or per-merged-token (ratio = merge^2) features."""
        in_rows = [r // ratio for r in book["out_rows"]]
        out_rows = [r // ratio for r in book["in_rows"]]
        y = _ListAllToAll.apply(self.group, in_rows, out_rows, feats)
        # rows come back in the order they were sent; undo the gather permutation at merged-token granularity
        idx = book["idx"].view(-1, ratio)[:, 0] // ratio if ratio > 1 else book["idx"]
        out = torch.empty_like(y)
        out.index_copy_(0, idx.to(y.device), y)
        return out
