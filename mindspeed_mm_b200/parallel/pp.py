"""Pipeline-parallel schedules over point-to-point sends (NCCL on GPUs, gloo on CPU).

``PipelineSchedule.run(micro_batches)`` executes one optimizer step's forwards and backwards on this stage:
  * ``1f1b``        warm-up of (pp - rank - 1) forwards, steady one-forward-one-backward, cool-down backwards
  * ``interleaved`` every rank holds ``v`` model chunks (virtual stages rank, rank+pp, ...); micro-batches advance
                    through chunks in groups of ``pp``, which shrinks the bubble by ``v``
                    (needs ``num_micro_batches % pp == 0``)
The reference takes both from Megatron (``get_forward_backward_func``, mindspeed_mm/training.py:750-765) and
only customises the tensor shapes it sends (wan_dit.py:525-570).  Activations travel forward and gradients
backward on two separate process groups, so each direction is an independent FIFO; sends are asynchronous
(``isend``) and overlap with the next compute, receives block just before their consumer.

``stage_fn(chunk, x_in, micro_batch) -> tensor`` runs one model chunk: ``x_in`` is None on the first virtual
stage; the last virtual stage returns the scalar loss of the micro-batch (already divided by the number of
micro-batches if that normalisation is wanted).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class PipelineSchedule:
    def __init__(self, stage_fn: Callable, pp_group, shape_fn: Callable[[dict], Tuple[int, ...]], dtype, device,
                 num_chunks: int = 1, fwd_group=None, bwd_group=None, after_backward: Optional[Callable[[], None]] = None):
        self.stage_fn, self.shape_fn, self.dtype, self.device = stage_fn, shape_fn, dtype, torch.device(device)
        self.group = pp_group
        self.pp = dist.get_world_size(pp_group) if pp_group is not None else 1
        self.rank = dist.get_rank(pp_group) if pp_group is not None else 0
        self.v = num_chunks
        ranks = dist.get_process_group_ranks(pp_group) if self.pp > 1 else [0]
        # independent channels for activations (forward) and gradients (backward)
        self.fwd_group = fwd_group if fwd_group is not None else pp_group
        self.bwd_group = bwd_group if bwd_group is not None else pp_group
        self.next = ranks[(self.rank + 1) % self.pp]
        self.prev = ranks[(self.rank - 1) % self.pp]
        self._pending: List = []
        self.after_backward = after_backward

    # -------------------------------------------------------------------------------------- p2p
    def _is_first(self, chunk):   # first virtual stage overall
        return self.rank == 0 and chunk == 0

    def _is_last(self, chunk):
        return self.rank == self.pp - 1 and chunk == self.v - 1

    def _recv(self, src, group, shape):
        t = torch.empty(shape, dtype=self.dtype, device=self.device)
        dist.recv(t, src=src, group=group)
        return t

    def _send(self, t, dst, group):
        self._pending.append((dist.isend(t.contiguous(), dst=dst, group=group), t))

    def _drain(self):
        for w, _ in self._pending:
            w.wait()
        self._pending = []

    # -------------------------------------------------------------------------------------- steps
    def _forward(self, chunk, mb, store):
        x = None
        if not self._is_first(chunk):
            x = self._recv(self.prev, self.fwd_group, self.shape_fn(mb)).requires_grad_()
        out = self.stage_fn(chunk, x, mb)
        if not self._is_last(chunk):
            self._send(out.detach(), self.next, self.fwd_group)
        store.append((x, out))
        return out

    def _backward(self, chunk, mb, store):
        x, out = store.pop(0)
        if self._is_last(chunk):
            out.backward()
        else:
            g = self._recv(self.next, self.bwd_group, tuple(out.shape))
            torch.autograd.backward(out, g)
        if not self._is_first(chunk):
            self._send(x.grad, self.prev, self.bwd_group)
        if self.after_backward is not None:
            self.after_backward()

    # -------------------------------------------------------------------------------------- schedules
    def run(self, micro_batches: Sequence[dict], schedule: str = "1f1b") -> List[torch.Tensor]:
        if self.pp == 1 and self.v == 1:
            losses = []
            for mb in micro_batches:
                loss = self.stage_fn(0, None, mb)
                loss.backward()
                if self.after_backward is not None:
                    self.after_backward()
                losses.append(loss.detach())
            return losses
        if schedule == "interleaved" or self.v > 1:
            return self._run_interleaved(micro_batches)
        return self._run_1f1b(micro_batches)

    def _run_1f1b(self, mbs):
        n = len(mbs)
        warm = min(self.pp - self.rank - 1, n)
        store: List = []
        losses = []
        fi = bi = 0
        for _ in range(warm):
            out = self._forward(0, mbs[fi], store)
            fi += 1
        for _ in range(n - warm):
            out = self._forward(0, mbs[fi], store)
            if self._is_last(0):
                losses.append(out.detach())
            fi += 1
            self._backward(0, mbs[bi], store)
            bi += 1
        for _ in range(warm):
            self._backward(0, mbs[bi], store)
            bi += 1
        self._drain()
        return losses

    def _run_interleaved(self, mbs):
        n, pp, v = len(mbs), self.pp, self.v
        if n % pp:
            raise ValueError(f"interleaved schedule needs num_micro_batches ({n}) divisible by pp ({pp})")
        total = n * v

        def fwd_item(k):        # k-th forward of this rank -> (chunk, micro-batch index)
            grp, r = divmod(k, pp * v)
            return r // pp, grp * pp + r % pp

        def bwd_item(k):
            grp, r = divmod(k, pp * v)
            return v - 1 - r // pp, grp * pp + r % pp

        warm = min((pp - self.rank - 1) * 2 + (v - 1) * pp, total)
        stores = [[] for _ in range(v)]
        losses = []
        for k in range(warm):
            c, i = fwd_item(k)
            self._forward(c, mbs[i], stores[c])
        for k in range(total - warm):
            c, i = fwd_item(warm + k)
            out = self._forward(c, mbs[i], stores[c])
            if self._is_last(c):
                losses.append(out.detach())
            cb, ib = bwd_item(k)
            self._backward(cb, mbs[ib], stores[cb])
        for k in range(total - warm, total):
            cb, ib = bwd_item(k)
            self._backward(cb, mbs[ib], stores[cb])
        if self.rank == pp - 1 and not losses:      # all forwards of the last stage happened during warm-up
            pass
        self._drain()
        return losses


def bubble_fraction(pp: int, num_micro_batches: int, num_chunks: int = 1) -> float:
    """Idle fraction of the classic schedules: (pp - 1) / (v * m + pp - 1)."""
    return (pp - 1) / (num_chunks * num_micro_batches + pp - 1)


def split_layers(num_layers: int, pp: int, given: Optional[Sequence[int]] = None) -> List[int]:
    """``pipeline_num_layers`` if given (must add up), else as even as possible with the remainder up front."""
    if given is not None:
        given = list(given)
        if len(given) != pp or sum(given) != num_layers:
            raise ValueError(f"pipeline_num_layers {given} must have {pp} entries adding up to {num_layers}")
        return given
    base, rem = divmod(num_layers, pp)
    return [base + (1 if r < rem else 0) for r in range(pp)]
