"""Megatron-style tensor parallelism with sequence parallelism.

Layers: ``ColumnParallelLinear`` (output features split; with sequence parallel the input is all-gathered
along the sequence first), ``RowParallelLinear`` (input features split; output reduce-scattered along the
sequence, or all-reduced without sequence parallel), ``VocabParallelEmbedding`` and the vocabulary-parallel
cross entropy (max / sum-exp / target logit each all-reduced over the group, never gathering [T, V]).
The reference uses Megatron's implementations of the same layers (mindspeed_mm/models/common/attention.py:296-389,
vlm_model.py:409-566).  With sequence parallelism on the native tier (CUDA, bf16, rows per rank a multiple of 128) the
two linears run the fused kernels of ``comm/fused.py`` in both directions: ``AllGatherLinear`` (the sequence all-gather
happens inside the column GEMM; its backward pushes the data gradient's row blocks to their owners) and
``RowParallelLinearRS`` (the row GEMM's epilogue is the reduce-scatter; its backward gathers the gradient rows inside
the GEMM).  Everything else (CPU / gloo, the library tier, no sequence parallelism, odd shapes) uses
``torch.distributed`` collectives around the GEMMs.  All tensors are [T, H] (packed tokens first).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


def _ws(group):
    return dist.get_world_size(group) if group is not None and dist.is_initialized() else 1


def _rk(group):
    return dist.get_rank(group) if group is not None and dist.is_initialized() else 0


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer without sequence parallel)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel layer without sequence parallel)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherSeq(torch.autograd.Function):
    """All-gather along dim 0 forward, reduce-scatter backward (sequence parallel -> tensor parallel region)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = x.new_empty(w * x.shape[0], *x.shape[1:])
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter0(g, ctx.group), None


class _ScatterSeq(torch.autograd.Function):
    """Reduce-scatter along dim 0 forward, all-gather backward (tensor parallel -> sequence parallel region)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter0(x, group)

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = g.new_empty(w * g.shape[0], *g.shape[1:])
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def _reduce_scatter0(x, group):
    w, r = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    out = x.new_empty(x.shape[0] // w, *x.shape[1:])
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x, group=group)
    else:                                   # gloo has no reduce_scatter
        y = x.clone()
        dist.all_reduce(y, group=group)
        out.copy_(y.chunk(w)[r])
    return out


def _fused_sp(x: torch.Tensor, group, rows_local: int, width: int) -> bool:
    """Fused GEMM + collective kernels apply: native tier, CUDA bf16 [T, H] input, 128-row blocks per rank."""
    if x.dim() != 2 or not x.is_cuda or _ws(group) > 8 or rows_local % 128 or width % 64:
        return False
    from ..comm import fused
    return fused.fused_supported(x)


def gather_sequence(x, group):
    return x if _ws(group) == 1 else _GatherSeq.apply(x, group)


def scatter_sequence(x, group):
    return x if _ws(group) == 1 else _ScatterSeq.apply(x, group)


def split_sequence(x, group):
    """Plain split (no reduction) of a replicated tensor along dim 0; backward all-gathers."""
    from .cp.split import split_forward_gather_backward
    return split_forward_gather_backward(x, group, dim=0)


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features, out_features, group, bias=True, sequence_parallel=False, gather_output=False):
        super().__init__()
        self.group, self.tp, self.sp, self.gather_output = group, _ws(group), sequence_parallel, gather_output
        if out_features % self.tp:
            raise ValueError(f"out_features {out_features} not divisible by tp {self.tp}")
        self.weight = nn.Parameter(torch.empty(out_features // self.tp, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features // self.tp)) if bias else None

    def forward(self, x):
        if self.tp > 1 and self.sp and not self.gather_output and _fused_sp(x, self.group, x.shape[0], x.shape[1]) \
                and self.weight.shape[0] % 8 == 0:
            from ..comm import fused
            return fused.shared(fused.AllGatherLinear, self.group, x.device, x.shape[0], x.shape[1])(x, self.weight, self.bias)
        if self.tp > 1:
            x = gather_sequence(x, self.group) if self.sp else _CopyToTP.apply(x, self.group)
        y = ops.linear(x, self.weight, self.bias)
        if self.gather_output and self.tp > 1:
            from .cp.split import gather_forward_split_backward
            y = gather_forward_split_backward(y, self.group, dim=-1)
        return y


class RowParallelLinear(nn.Module):
    def __init__(self, in_features, out_features, group, bias=True, sequence_parallel=False):
        super().__init__()
        self.group, self.tp, self.sp = group, _ws(group), sequence_parallel
        if in_features % self.tp:
            raise ValueError(f"in_features {in_features} not divisible by tp {self.tp}")
        self.weight = nn.Parameter(torch.empty(out_features, in_features // self.tp))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None      # added once, after the reduction

    def forward(self, x):
        if self.tp > 1 and self.sp and x.dim() == 2 and x.shape[0] % self.tp == 0 and x.shape[1] % 8 == 0 and \
                _fused_sp(x, self.group, x.shape[0] // self.tp, self.weight.shape[0]):
            from ..comm import fused
            y = fused.shared(fused.RowParallelLinearRS, self.group, x.device, x.shape[0], self.weight.shape[0])(x, self.weight)
            return y if self.bias is None else y + self.bias
        y = ops.linear(x, self.weight, None)
        if self.tp > 1:
            y = scatter_sequence(y, self.group) if self.sp else _ReduceFromTP.apply(y, self.group)
        return y if self.bias is None else y + self.bias


class VocabParallelEmbedding(nn.Module):
    def __init__(self, vocab, dim, group, sequence_parallel=False):
        super().__init__()
        self.group, self.tp, self.sp = group, _ws(group), sequence_parallel
        self.per = vocab // self.tp
        self.lo = _rk(group) * self.per
        self.weight = nn.Parameter(torch.empty(self.per, dim))

    def forward(self, ids):
        if self.tp == 1:
            return F.embedding(ids, self.weight)
        mask = (ids < self.lo) | (ids >= self.lo + self.per)
        local = (ids - self.lo).masked_fill(mask, 0)
        out = F.embedding(local, self.weight).masked_fill(mask.unsqueeze(-1), 0.0)
        return scatter_sequence(out, self.group) if self.sp else _ReduceFromTP.apply(out, self.group)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, group, lo, ignore_index):
        lf = logits.float()
        mx = lf.max(-1).values
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        ex = torch.exp(lf - mx[:, None])
        se = ex.sum(-1)
        dist.all_reduce(se, group=group)
        per = logits.shape[1]
        valid = labels != ignore_index
        mine = valid & (labels >= lo) & (labels < lo + per)
        loc = (labels - lo).clamp(0, per - 1)
        tgt = torch.where(mine, lf.gather(1, loc[:, None]).squeeze(1), torch.zeros_like(mx))
        dist.all_reduce(tgt, group=group)
        loss = (torch.log(se) + mx - tgt) * valid
        ctx.save_for_backward(ex / se[:, None], loc, mine, valid)
        ctx.dtype = logits.dtype
        return loss.sum()

    @staticmethod
    def backward(ctx, g):
        p, loc, mine, valid = ctx.saved_tensors
        p = p.clone()
        p[torch.arange(p.shape[0], device=p.device), loc] -= mine.to(p.dtype)
        p *= valid[:, None]
        return (p * g).to(ctx.dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits_local, labels, group, ignore_index: int = -100):
    """Sum of token CE where ``logits_local`` is this rank's vocabulary slice [T, V/tp]."""
    if _ws(group) == 1:
        return F.cross_entropy(logits_local.float(), labels, ignore_index=ignore_index, reduction="sum")
    lo = _rk(group) * logits_local.shape[1]
    out = _VocabParallelCE.apply(logits_local, labels, group, lo, ignore_index)
    return out
