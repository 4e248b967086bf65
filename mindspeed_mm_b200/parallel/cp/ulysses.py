"""Ulysses sequence parallelism: all-to-all between "sequence-sharded, all heads" and "full sequence,
head-sharded" layouts around the attention core.

Reference: mindspeed_mm/fsdp/distributed/context_parallel/communication.py:78-128,175-220 (aligned and
unaligned ``all_to_all``), mindspeed_mm/fsdp/ops/flash_attn/flash_attn.py:281-295 (KV heads are replicated
when the group is larger than the number of KV heads) and models/common/attention.py (UlyssesContextAttention).
Tensors are [B, S_local, N, D].  The functions here are the collective form (``dist.all_to_all_single`` / ``all_to_all``):
CPU / gloo runs, the library tier, unaligned sequences.  On the native tier the Wan DiT does not call them for its
self-attention: the scatter is the epilogue of the QKV GEMM and the gather the operand fetch of the output projection
(``comm/fused.py``, used from ``models/wan.py: WanSelfAttention._forward_fused``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .split import cal_split_sizes


def _a2a(x: torch.Tensor, scatter_dim: int, gather_dim: int, group, scatter_sizes: Sequence[int],
         gather_sizes: Sequence[int]) -> torch.Tensor:
    """Scatter ``scatter_dim`` over the group and gather ``gather_dim`` (sizes may be uneven)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    parts = [p.contiguous() for p in torch.split(x, list(scatter_sizes), dim=scatter_dim)]
    outs = []
    for r in range(world):
        shape = list(parts[rank].shape)
        shape[gather_dim] = gather_sizes[r]
        outs.append(x.new_empty(shape))
    if len(set(scatter_sizes)) == 1 and len(set(gather_sizes)) == 1:
        inp = torch.stack(parts, 0)
        out = torch.empty_like(inp)
        dist.all_to_all_single(out, inp, group=group)
        outs = list(out.unbind(0))
    else:
        dist.all_to_all(outs, parts, group=group)
    return torch.cat(outs, dim=gather_dim)


class _SeqAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scatter_dim, gather_dim, group, scatter_sizes, gather_sizes):
        ctx.args = (scatter_dim, gather_dim, group, scatter_sizes, gather_sizes)
        return _a2a(x, scatter_dim, gather_dim, group, scatter_sizes, gather_sizes)

    @staticmethod
    def backward(ctx, g):
        scatter_dim, gather_dim, group, scatter_sizes, gather_sizes = ctx.args
        return _a2a(g, gather_dim, scatter_dim, group, gather_sizes, scatter_sizes), None, None, None, None, None


def all_to_all(x, group, scatter_dim: int, gather_dim: int, scatter_sizes=None, gather_sizes=None):
    """Differentiable all-to-all.  Without explicit sizes both dims are split near-evenly; pass
    ``gather_sizes`` = every rank's local length for unaligned sequences."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    world = dist.get_world_size(group)
    if scatter_sizes is None:
        scatter_sizes = cal_split_sizes(x.shape[scatter_dim], world)
    if gather_sizes is None:
        gather_sizes = [x.shape[gather_dim]] * world
    return _SeqAllToAll.apply(x, scatter_dim, gather_dim, group, list(scatter_sizes), list(gather_sizes))


def repeat_kv_for_ulysses(k: torch.Tensor, v: torch.Tensor, world: int):
    """When the group is larger than the KV head count, replicate KV heads so each rank gets at least one."""
    nkv = k.shape[2]
    if nkv >= world:
        return k, v
    rep = world // nkv
    return k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)


def ulysses_attention(attn_fn, q, k, v, group, seq_sizes: Optional[List[int]] = None, **kw):
    """``attn_fn(q, k, v, **kw)`` on full sequences with 1/P of the heads; inputs/outputs are sequence-sharded
    [B, S_local, N, D].  ``seq_sizes``: per-rank local sequence lengths when they differ."""
    if group is None or dist.get_world_size(group) == 1:
        return attn_fn(q, k, v, **kw)
    world = dist.get_world_size(group)
    k, v = repeat_kv_for_ulysses(k, v, world)
    q = all_to_all(q, group, scatter_dim=2, gather_dim=1, gather_sizes=seq_sizes)
    k = all_to_all(k, group, scatter_dim=2, gather_dim=1, gather_sizes=seq_sizes)
    v = all_to_all(v, group, scatter_dim=2, gather_dim=1, gather_sizes=seq_sizes)
    o = attn_fn(q, k, v, **kw)
    return all_to_all(o, group, scatter_dim=1, gather_dim=2, scatter_sizes=seq_sizes)
