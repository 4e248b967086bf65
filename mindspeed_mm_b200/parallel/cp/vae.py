"""Context parallelism over the frame axis for the causal 3-D autoencoders.

A clip of ``1 + c * m`` frames (``c`` = temporal compression) is split along time: rank 0 holds ``1 + c * m_0`` frames, every
other rank ``c * m_r``, so that after each temporal stride-2 stage the pieces still line up (rank 0: ``1 + (c/2) m_0``,
others ``(c/2) m_r``).  Three things need the neighbours:

* causal temporal convolutions: the ``kt - 1`` frames in front of a rank's piece are the tail of its predecessor's piece
  (rank 0 replicates its first frame, as the single-device module does) -> ``halo_front``;
* GroupNorm: mean / variance are taken over all frames of the clip -> ``cp_group_norm`` (sums all-reduced, differentiable);
* the temporal up-sampling of the decoder treats the clip's first latent frame specially (it stands for one pixel frame):
  only rank 0 has it.

Reference: mindspeed_mm/models/ae/contextparallel_causalvae.py and mindspeed_mm/models/common/conv.py
(``ContextParallelCausalConv3d``: send / recv of the last ``kt - 1`` frames), mindspeed_mm/models/common/normalize.py
(group norm with statistics reduced over the context-parallel group).

``apply_context_parallel(vae, group)`` patches a ``CausalVAE3D`` in place; ``split_frames`` / ``gather_frames`` move a clip
in and out of the split layout.  Collectives are plain ``torch.distributed`` calls (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------- layout
def frame_counts(total: int, world: int, compression: int) -> List[int]:
    """Frames per rank for a clip of ``1 + compression * m`` frames: blocks of ``compression`` frames dealt as evenly as
    possible, the lone first frame added to rank 0."""
    if (total - 1) % compression:
        raise ValueError(f"{total} frames is not 1 + k * {compression}")
    blocks = (total - 1) // compression
    if blocks < world:
        raise ValueError(f"{blocks} blocks of {compression} frames cannot be split over {world} ranks")
    per = [blocks // world + (1 if r < blocks % world else 0) for r in range(world)]
    return [compression * p + (1 if r == 0 else 0) for r, p in enumerate(per)]


def split_frames(x: torch.Tensor, group, compression: int, dim: int = 2) -> torch.Tensor:
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    counts = frame_counts(x.shape[dim], world, compression)
    start = sum(counts[:rank])
    return x.narrow(dim, start, counts[rank]).contiguous()


class _GatherFrames(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, counts, dim):
        ctx.group, ctx.counts, ctx.dim = group, counts, dim
        rank = dist.get_rank(group)
        parts = []
        for r, n in enumerate(counts):
            shape = list(x.shape)
            shape[dim] = n
            parts.append(x.contiguous() if r == rank else x.new_empty(shape))
        dist.all_gather(parts, x.contiguous(), group=group) if len(set(counts)) == 1 else _uneven_all_gather(parts, x, group)
        return torch.cat(parts, dim)

    @staticmethod
    def backward(ctx, g):
        rank = dist.get_rank(ctx.group)
        start = sum(ctx.counts[:rank])
        return g.narrow(ctx.dim, start, ctx.counts[rank]).contiguous(), None, None, None


def _uneven_all_gather(parts, x, group):
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    for r in range(world):
        src = dist.get_global_rank(group, r) if group is not None else r
        buf = x.contiguous() if r == rank else parts[r]
        dist.broadcast(buf, src=src, group=group)
        parts[r] = buf


def gather_frames(x: torch.Tensor, group, counts: List[int], dim: int = 2) -> torch.Tensor:
    """Concatenate the ranks' pieces along ``dim`` (every rank gets the whole clip; the backward keeps its own slice)."""
    return _GatherFrames.apply(x, group, list(counts), dim)


# ------------------------------------------------------------------------------------------------- halo
class _HaloFront(torch.autograd.Function):
    """[B, C, T, H, W] -> [B, C, n + T, H, W]: the predecessor's last ``n`` frames in front (rank 0: its first frame
    repeated ``n_first`` times).  Backward: the gradient of the borrowed frames travels back to their owner."""

    @staticmethod
    def forward(ctx, x, n, group, n_first):
        ctx.n, ctx.group, ctx.n_first = n, group, n_first
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ctx.rank, ctx.world = rank, world
        if x.shape[2] < n:
            raise ValueError(f"a rank holds {x.shape[2]} frames, fewer than the {n} its successor needs")
        tail = x[:, :, -n:].contiguous()
        recv = torch.empty_like(tail)
        _shift(tail if rank < world - 1 else None, recv if rank > 0 else None, +1, group)
        if rank == 0:
            recv = x[:, :, :1].expand(-1, -1, n_first, -1, -1)
        return torch.cat([recv, x], 2)

    @staticmethod
    def backward(ctx, g):
        n, rank, world = ctx.n, ctx.rank, ctx.world
        front = ctx.n_first if rank == 0 else n
        gx = g[:, :, front:].clone()
        ghalo = g[:, :, :front].contiguous()
        back = gx.new_empty(gx.shape[:2] + (n,) + gx.shape[3:])
        _shift(ghalo if rank > 0 else None, back if rank < world - 1 else None, -1, ctx.group)
        if rank < world - 1:
            gx[:, :, -n:] += back
        if rank == 0:
            gx[:, :, :1] += ghalo.sum(2, keepdim=True)
        return gx, None, None, None


def _shift(send: Optional[torch.Tensor], recv: Optional[torch.Tensor], direction: int, group) -> None:
    """Every rank sends to ``rank + direction`` and receives from ``rank - direction`` (ends of the line skip one side)."""
    rank = dist.get_rank(group)
    peer = lambda r: dist.get_global_rank(group, r) if group is not None else r       # noqa: E731
    ops = []
    if send is not None:
        ops.append(dist.P2POp(dist.isend, send, peer(rank + direction), group))
    if recv is not None:
        ops.append(dist.P2POp(dist.irecv, recv, peer(rank - direction), group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


def halo_front(x: torch.Tensor, n: int, group, n_first: Optional[int] = None) -> torch.Tensor:
    """``n`` frames borrowed from the predecessor; rank 0 replicates its first frame ``n_first`` (default ``n``) times.  A
    stride-``s`` convolution of temporal kernel ``kt`` borrows ``kt - s`` frames (its first window on a later rank starts
    that far into the predecessor's piece) while rank 0 keeps the full causal pad ``kt - 1``."""
    return _HaloFront.apply(x, n, group, n if n_first is None else n_first) if max(n, n_first or 0) > 0 else x


# ------------------------------------------------------------------------------------------------- group norm
class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def cp_group_norm(n: nn.GroupNorm, x: torch.Tensor, group) -> torch.Tensor:
    """GroupNorm of module ``n`` with statistics over the frames of ALL ranks of ``group``."""
    B, C = x.shape[:2]
    xg = x.reshape(B, n.num_groups, -1).to(torch.float64 if x.dtype == torch.float64 else torch.float32)
    stats = torch.stack([xg.sum(-1), (xg * xg).sum(-1), torch.full_like(xg[..., 0], xg.shape[-1])])
    stats = _AllReduceSum.apply(stats, group)
    mean = stats[0] / stats[2]
    var = (stats[1] / stats[2] - mean * mean).clamp_min(0)
    y = ((xg - mean[..., None]) * torch.rsqrt(var[..., None] + n.eps)).reshape(x.shape).to(x.dtype)
    shape = (1, C) + (1,) * (x.dim() - 2)
    return y * n.weight.view(shape) + n.bias.view(shape) if n.affine else y


# ------------------------------------------------------------------------------------------------- module patching
def apply_context_parallel(vae: nn.Module, group) -> nn.Module:
    """Patch a ``models.ae.kl_vae.CausalVAE3D`` in place for inputs split along time over ``group`` (no-op for a group of
    one).  Parameter names do not change; gradients of the (replicated) parameters are partial per rank and must be summed
    over the group like any data-parallel gradient."""
    from ...models.ae import kl_vae
    if group is None or dist.get_world_size(group) == 1:
        return vae
    rank = dist.get_rank(group)

    def conv_forward(self, x):
        if self.kt > 1:
            if not self.causal:
                raise NotImplementedError("context parallelism covers the causal temporal convolutions")
            x = halo_front(x, self.kt - 1, group)
        return self.conv(x)

    def down_forward(self, x):
        x = F.pad(x, (0, 1, 0, 1))
        if self.kt > 1:
            if rank > 0 and x.shape[2] % 2:
                raise ValueError("ranks after the first must hold an even number of frames before a temporal stride-2 stage")
            x = halo_front(x, self.kt - 2, group, n_first=self.kt - 1)
        return self.conv(x)

    def up_forward(self, x):
        B, C, T, H, W = x.shape
        if self.time:
            if rank == 0 and T > 1:
                x = torch.cat([x[:, :, :1], x[:, :, 1:].repeat_interleave(2, 2)], 2)
            elif rank > 0:                      # no lone first frame here: every latent frame stands for two
                x = x.repeat_interleave(2, 2)
        x = F.interpolate(x.flatten(1, 2).reshape(B, C * x.shape[2], H, W), scale_factor=2.0, mode="nearest").reshape(B, C, -1, 2 * H, 2 * W)
        return self.conv(x)

    for m in vae.modules():
        if isinstance(m, nn.GroupNorm):
            m.forward = (lambda n: lambda x: cp_group_norm(n, x, group))(m)
        elif isinstance(m, kl_vae.Conv):
            m.forward = conv_forward.__get__(m)
        elif isinstance(m, kl_vae.Down):
            m.forward = down_forward.__get__(m)
        elif isinstance(m, kl_vae.Up):
            m.forward = up_forward.__get__(m)
    vae.cp_group = group
    return vae
