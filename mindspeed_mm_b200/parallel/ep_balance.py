"""Expert-load balancing by duplicating hot experts.

Given the per-expert token counts of the last step, ``plan_duplicates`` greedily picks up to ``max_dup`` hot
experts per rank to replicate on the least loaded ranks and splits the hot expert's tokens between owner and
replica; ``apply_plan`` rewrites a routing table (expert id -> (rank, local slot)) accordingly.  The reference
does the same with a numba planner and overlaps the weight copies with the permute
(mindspeed_mm/fsdp/distributed/expert_parallel/ep_balance/greedy_dup_experts_planner.py:265-363,
greedy_dup_experts_executor.py:6-197); ``exchange_duplicates`` moves replica weights with isend/irecv (NCCL p2p).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class DupPlan:
    # (expert, src_rank, dst_rank, fraction of the expert's tokens that move to dst)
    moves: List[Tuple[int, int, int, float]]
    loads_before: List[float]
    loads_after: List[float]


def plan_duplicates(expert_tokens: Sequence[float], ep: int, max_dup: int = 2) -> DupPlan:
    E = len(expert_tokens)
    per = E // ep
    owner = [e // per for e in range(E)]
    loads = [0.0] * ep
    for e, c in enumerate(expert_tokens):
        loads[owner[e]] += c
    before = list(loads)
    remaining = {e: float(c) for e, c in enumerate(expert_tokens)}
    dups = [0] * ep
    moves: List[Tuple[int, int, int, float]] = []
    for _ in range(ep * max_dup):
        src = max(range(ep), key=lambda r: loads[r])
        dst = min((r for r in range(ep) if dups[r] < max_dup), key=lambda r: loads[r], default=None)
        if dst is None or dst == src or loads[src] - loads[dst] < 1e-9:
            break
        cand = [e for e in range(E) if owner[e] == src and remaining[e] > 0]
        if not cand:
            break
        hot = max(cand, key=lambda e: remaining[e])
        shift = min(remaining[hot], (loads[src] - loads[dst]) / 2)
        if shift <= 0:
            break
        moves.append((hot, src, dst, shift / max(float(expert_tokens[hot]), 1e-9)))
        remaining[hot] -= shift
        loads[src] -= shift
        loads[dst] += shift
        dups[dst] += 1
    return DupPlan(moves, before, loads)


def apply_plan(topk_ids: torch.Tensor, plan: DupPlan, num_experts: int) -> torch.Tensor:
    """Return routed ids where a fraction of each duplicated expert's slots point at a virtual replica id
    ``num_experts + i`` (i = index of the move); the dispatcher maps virtual ids to (dst rank, replica slot)."""
    out = topk_ids.clone()
    flat = out.view(-1)
    orig = topk_ids.reshape(-1)
    taken = {}
    for i, (e, _, _, frac) in enumerate(plan.moves):
        idx = (orig == e).nonzero(as_tuple=True)[0]          # fractions refer to the expert's ORIGINAL slots
        n = int(round(frac * idx.numel()))
        start = taken.get(e, 0)
        if n:
            flat[idx[start:start + n]] = num_experts + i
        taken[e] = start + n
    return out


def exchange_duplicates(weights: Dict[str, torch.Tensor], plan: DupPlan, ep_group, experts_per_rank: int):
    """Ship the duplicated experts' weights from owner to replica rank (async p2p); returns {move index: tensors}."""
    rank = dist.get_rank(ep_group)
    reqs, recv = [], {}
    for i, (e, src, dst, _) in enumerate(plan.moves):
        local = e % experts_per_rank
        for name, w in weights.items():
            if rank == src:
                reqs.append(dist.isend(w[local].contiguous(), dist.get_global_rank(ep_group, dst), group=ep_group))
            elif rank == dst:
                buf = torch.empty_like(w[0])
                reqs.append(dist.irecv(buf, dist.get_global_rank(ep_group, src), group=ep_group))
                recv.setdefault(i, {})[name] = buf
    for r in reqs:
        r.wait()
    return recv
