"""Context parallelism for PACKED sequences (the TND layout with document boundaries): all-gather of keys / values.

The packed token stream of ``T`` tokens (several documents, boundaries in ``cu_seqlens``) is cut into ``W`` equal,
contiguous chunks, one per rank.  Queries stay local; keys and values (few heads under GQA) are all-gathered over the
context-parallel group, and every rank runs ONE varlen attention call of its query chunk against the contiguous key
range it can see: from the start of the first document that overlaps its chunk to the end of its chunk.  Document
boundaries inside that range become the segments of the call, and the causal mask is the bottom-right aligned one of each
segment (a document that began on an earlier rank has more keys than queries here), so no mask tensor is built.

Reference: the packed ("TND" / end-of-document reset) context-parallel strategies of
mindspeed_mm/patchs/ring_attn_patch.py:37-66 and mindspeed_mm/fsdp/distributed/context_parallel (cu_seqlens-aware splits).
The gradient of the gathered keys / values is reduce-scattered back to the owners.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ... import ops


class _AllGatherTokens(torch.autograd.Function):
    """[T / W, ...] -> [T, ...] along dim 0; backward: reduce-scatter (sum) of the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group)
        out = x.new_empty((W * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        W = dist.get_world_size(ctx.group)
        out = g.new_empty((g.shape[0] // W,) + tuple(g.shape[1:]))
        if dist.get_backend(ctx.group) == "gloo":          # no reduce-scatter on gloo: all-reduce and keep the own part
            g = g.contiguous().clone()
            dist.all_reduce(g, group=ctx.group)
            r = dist.get_rank(ctx.group)
            out = g[r * out.shape[0]:(r + 1) * out.shape[0]].clone()
        else:
            dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def chunk_plan(cu_seqlens: Sequence[int], world: int, rank: int) -> Tuple[int, int, List[int], List[int]]:
    """For rank ``rank``'s chunk ``[lo, hi)`` of the packed stream: ``(key_start, hi, cu_q, cu_k)`` where the keys are
    tokens ``[key_start, hi)`` and ``cu_q`` / ``cu_k`` are the segment boundaries relative to ``lo`` / ``key_start``."""
    cu = [int(c) for c in cu_seqlens]
    T = cu[-1]
    if T % world:
        raise ValueError(f"{T} packed tokens cannot be cut into {world} equal chunks (pad the pack)")
    per = T // world
    lo, hi = rank * per, (rank + 1) * per
    cu_q, cu_k, key_start = [0], [0], None
    for a, b in zip(cu[:-1], cu[1:]):
        qa, qb = max(a, lo), min(b, hi)
        if qa >= qb:
            continue
        if key_start is None:
            key_start = a
        cu_q.append(qb - lo)
        cu_k.append(qb - key_start)
    return key_start if key_start is not None else lo, hi, cu_q, cu_k


def packed_attention(q, k, v, cu_seqlens, group, causal: bool = True, softmax_scale: Optional[float] = None):
    """q: [T / W, Nq, D]; k, v: [T / W, Nkv, D] (this rank's chunk of the packed stream); ``cu_seqlens``: boundaries of the
    WHOLE stream (the same on every rank).  Returns the attention output of the local queries, [T / W, Nq, D]."""
    if group is None or dist.get_world_size(group) == 1:
        cu = torch.as_tensor(cu_seqlens, dtype=torch.int32, device=q.device)
        mx = int((cu[1:] - cu[:-1]).max())
        return ops.attention_varlen(q, k, v, cu, cu, mx, mx, causal=causal, softmax_scale=softmax_scale)
    if not causal:
        raise NotImplementedError("non-causal packed attention needs the keys after the chunk as well; use Ulysses there")
    W, r = dist.get_world_size(group), dist.get_rank(group)
    kv = _AllGatherTokens.apply(torch.stack([k, v], 1), group)          # [T, 2, Nkv, D]
    key_start, hi, cu_q, cu_k = chunk_plan(cu_seqlens, W, r)
    ks, vs = kv[key_start:hi, 0], kv[key_start:hi, 1]
    cq = torch.tensor(cu_q, dtype=torch.int32, device=q.device)
    ck = torch.tensor(cu_k, dtype=torch.int32, device=q.device)
    mq = max(b - a for a, b in zip(cu_q[:-1], cu_q[1:]))
    mk = max(b - a for a, b in zip(cu_k[:-1], cu_k[1:]))
    return ops.attention_varlen(q, ks.contiguous(), vs.contiguous(), cq, ck, mq, mk, causal=True, softmax_scale=softmax_scale)
