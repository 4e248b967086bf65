"""Sequence split / gather with autograd, aligned and unaligned, plus the zig-zag causal balance.

Reference: mindspeed_mm/fsdp/distributed/context_parallel/communication.py:131-290 (``cal_split_sizes``,
``split_forward_gather_backward``, ``gather_forward_split_backward``) and :760-926 (zig-zag / packed split).
``grad_scale``: "down" divides the gathered gradient by the group size, "up" multiplies (the reference's
convention for keeping loss scaling consistent when the loss is averaged over ranks).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def cal_split_sizes(dim_size: int, world_size: int) -> List[int]:
    """Near-even split: the first ``dim_size % world_size`` ranks get one extra element."""
    base, rem = divmod(dim_size, world_size)
    return [base + (1 if r < rem else 0) for r in range(world_size)]


def _rank_world(group):
    if group is None or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _all_gather_var(x: torch.Tensor, dim: int, sizes: Sequence[int], group) -> torch.Tensor:
    rank, world = _rank_world(group)
    if world == 1:
        return x
    x = x.contiguous()
    if len(set(sizes)) == 1:
        outs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(outs, x, group=group)
    else:
        mx = max(sizes)
        pad_shape = list(x.shape)
        pad_shape[dim] = mx
        buf = x.new_zeros(pad_shape)
        buf.narrow(dim, 0, x.shape[dim]).copy_(x)
        gathered = [torch.empty_like(buf) for _ in range(world)]
        dist.all_gather(gathered, buf, group=group)
        outs = [g.narrow(dim, 0, s) for g, s in zip(gathered, sizes)]
    return torch.cat(outs, dim=dim)


class _Split(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, sizes, group, grad_scale):
        rank, world = _rank_world(group)
        ctx.dim, ctx.sizes, ctx.group, ctx.grad_scale, ctx.world = dim, sizes, group, grad_scale, world
        start = sum(sizes[:rank])
        return x.narrow(dim, start, sizes[rank]).contiguous()

    @staticmethod
    def backward(ctx, g):
        if ctx.grad_scale == "up":
            g = g * ctx.world
        elif ctx.grad_scale == "down":
            g = g / ctx.world
        return _all_gather_var(g, ctx.dim, ctx.sizes, ctx.group), None, None, None, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, sizes, group, grad_scale):
        rank, world = _rank_world(group)
        ctx.dim, ctx.sizes, ctx.rank, ctx.grad_scale, ctx.world = dim, sizes, rank, grad_scale, world
        return _all_gather_var(x, dim, sizes, group)

    @staticmethod
    def backward(ctx, g):
        if ctx.grad_scale == "up":
            g = g * ctx.world
        elif ctx.grad_scale == "down":
            g = g / ctx.world
        start = sum(ctx.sizes[:ctx.rank])
        return g.narrow(ctx.dim, start, ctx.sizes[ctx.rank]).contiguous(), None, None, None, None


def split_forward_gather_backward(x, group, dim: int, grad_scale: Optional[str] = None, split_sizes=None):
    _, world = _rank_world(group)
    if world == 1:
        return x
    sizes = list(split_sizes) if split_sizes is not None else cal_split_sizes(x.shape[dim], world)
    return _Split.apply(x, dim, sizes, group, grad_scale)


def gather_forward_split_backward(x, group, dim: int, grad_scale: Optional[str] = None, gather_sizes=None):
    _, world = _rank_world(group)
    if world == 1:
        return x
    if gather_sizes is None:
        gather_sizes = [x.shape[dim]] * world
    return _Gather.apply(x, dim, list(gather_sizes), group, grad_scale)


def zigzag_indices(seq_len: int, world: int, rank: int) -> torch.Tensor:
    """Causal load balance: the sequence is cut into 2*world chunks and rank r takes chunks r and 2w-1-r."""
    if seq_len % (2 * world):
        raise ValueError(f"sequence length {seq_len} must be divisible by 2*cp ({2 * world}) for zig-zag split")
    c = seq_len // (2 * world)
    a = torch.arange(rank * c, (rank + 1) * c)
    b = torch.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c)
    return torch.cat([a, b])


def zigzag_split_packed(cu_seqlens: Sequence[int], world: int, rank: int) -> torch.Tensor:
    """Zig-zag split applied to every packed sub-sequence independently; returns token indices of ``rank``."""
    idx = []
    for s, e in zip(cu_seqlens[:-1], cu_seqlens[1:]):
        idx.append(zigzag_indices(int(e) - int(s), world, rank) + int(s))
    return torch.cat(idx)
