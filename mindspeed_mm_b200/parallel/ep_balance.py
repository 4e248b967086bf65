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


# ------------------------------------------------------------------------------------------ balanced dispatch
class _ShipReplicas(torch.autograd.Function):
    """Forward: every move's owner sends the hot expert's ``gate_up`` / ``down`` slices to the replica rank, which files
    them in its next free replica slot.  Backward: the replica sends the slot's weight gradients home and the owner adds
    them to the expert's own gradient, so the optimizer never sees the copies."""

    @staticmethod
    def forward(ctx, gate_up, down, moves, group, experts_per_rank, max_dup):
        rank = dist.get_rank(group)
        ctx.moves, ctx.group, ctx.per, ctx.max_dup, ctx.rank = moves, group, experts_per_rank, max_dup, rank
        rep_gu = gate_up.new_zeros((max_dup,) + tuple(gate_up.shape[1:]))
        rep_dn = down.new_zeros((max_dup,) + tuple(down.shape[1:]))
        reqs, slot = [], {}
        for e, src, dst, _ in moves:
            j = slot.get(dst, 0)
            slot[dst] = j + 1
            for w, rep in ((gate_up, rep_gu), (down, rep_dn)):
                if rank == src:
                    reqs.append(dist.isend(w[e % experts_per_rank].detach().contiguous(), dist.get_global_rank(group, dst),
                                           group=group))
                elif rank == dst:
                    reqs.append(dist.irecv(rep[j], dist.get_global_rank(group, src), group=group))
        for r in reqs:
            r.wait()
        return rep_gu, rep_dn

    @staticmethod
    def backward(ctx, g_gu, g_dn):
        rank, per = ctx.rank, ctx.per
        d_gu = d_dn = None
        reqs, adds, slot = [], [], {}
        for e, src, dst, _ in ctx.moves:
            j = slot.get(dst, 0)
            slot[dst] = j + 1
            for which, g in ((0, g_gu), (1, g_dn)):
                if rank == dst:
                    reqs.append(dist.isend(g[j].contiguous(), dist.get_global_rank(ctx.group, src), group=ctx.group))
                elif rank == src:
                    buf = torch.empty_like(g[0])
                    reqs.append(dist.irecv(buf, dist.get_global_rank(ctx.group, dst), group=ctx.group))
                    adds.append((which, e % per, buf))
        for r in reqs:
            r.wait()
        if adds:
            d_gu = g_gu.new_zeros((per,) + tuple(g_gu.shape[1:]))
            d_dn = g_dn.new_zeros((per,) + tuple(g_dn.shape[1:]))
            for which, local, buf in adds:
                (d_gu if which == 0 else d_dn)[local] += buf
        return d_gu, d_dn, None, None, None, None


def slot_table(plan: DupPlan, num_experts: int, ep: int, max_dup: int) -> torch.Tensor:
    """Expert id (real, then one virtual id per move) -> global slot, when every rank holds ``per + max_dup`` slots:
    its own experts first, then its replica slots in the order of the moves that target it."""
    per = num_experts // ep
    width = per + max_dup
    table = [(e // per) * width + e % per for e in range(num_experts)]
    used = {}
    for _, _, dst, _ in plan.moves:
        j = used.get(dst, 0)
        used[dst] = j + 1
        table.append(dst * width + per + j)
    return torch.tensor(table, dtype=torch.long)


def balanced_forward(dispatch_fn, tokens, topk_ids, probs, gate_up, down, num_experts: int, group, max_dup: int = 2):
    """Expert-parallel MoE forward with hot experts duplicated for this call: count the tokens per expert over the whole
    expert-parallel group, plan the moves, ship the replicas, rewrite the routing to slots and run ``dispatch_fn`` (any
    of the dispatchers of ``parallel/ep.py``) over ``per + max_dup`` slots per rank.  Same result as the unbalanced call;
    the busiest rank gets fewer rows."""
    ep = dist.get_world_size(group)
    counts = torch.bincount(topk_ids.reshape(-1), minlength=num_experts).float()
    dist.all_reduce(counts, group=group)
    plan = plan_duplicates(counts.tolist(), ep, max_dup)
    if not plan.moves:
        return dispatch_fn(tokens, topk_ids, probs, gate_up, down, num_experts, group), plan
    per = num_experts // ep
    rep_gu, rep_dn = _ShipReplicas.apply(gate_up, down, plan.moves, group, per, max_dup)
    # the split of a hot expert's tokens must be decided once for the whole group: take the fraction of every rank's
    # own slots (each rank moves the same share of what it routes there)
    virt = apply_plan(topk_ids, plan, num_experts)
    slots = slot_table(plan, num_experts, ep, max_dup).to(topk_ids.device)[virt]
    out = dispatch_fn(tokens, slots, probs, torch.cat([gate_up, rep_gu]), torch.cat([down, rep_dn]),
                      ep * (per + max_dup), group)
    return out, plan
