"""Hybrid context parallelism (Ulysses x ring, "USP") and chunked Ulysses attention (FPDT).

* ``usp_attention``: inside the Ulysses group the heads are scattered and the sequence gathered (all-to-all), and the
  ring group walks the K/V blocks of the gathered sub-sequences.  The reference selects this with
  ``--context-parallel-algo hybrid_cp_algo --ulysses-degree-in-cp`` (mindspeed_mm/models/common/attention.py:50-79)
  and ``ulysses x ring`` mesh dims on the native path (fsdp/distributed/parallel_state.py:53-67,
  fsdp/ops/flash_attn/flash_attn.py:343-379).  Rank layout: the Ulysses group is the inner (fastest) dimension, so
  its all-to-alls stay among neighbouring GPUs.
* ``usp_local_indices``: which tokens of the full sequence a rank holds -- zig-zag halves across the ring ranks
  when attention is causal (balanced work), a contiguous slice across the Ulysses ranks inside each ring chunk.
* ``fpdt_attention``: Ulysses attention computed one query chunk at a time, so only one chunk of scores /
  gathered queries is alive; gathered K/V chunks may be parked in pinned host memory between uses
  (mindspeed_mm/models/common/fpdt_layer.py:101-748).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ... import ops
from .ring import ring_attention
from .split import zigzag_indices
from .ulysses import all_to_all, repeat_kv_for_ulysses, ulysses_attention


def usp_local_indices(seq_len: int, ring_world: int, ring_rank: int, uly_world: int, uly_rank: int,
                      causal: bool) -> torch.Tensor:
    if causal:
        ring_idx = zigzag_indices(seq_len, ring_world, ring_rank)
    else:
        n = seq_len // ring_world
        ring_idx = torch.arange(ring_rank * n, (ring_rank + 1) * n)
    m = ring_idx.numel() // uly_world
    return ring_idx[uly_rank * m:(uly_rank + 1) * m]


def usp_attention(q, k, v, ulysses_group, ring_group, causal: bool = False, softmax_scale: Optional[float] = None):
    """q [B, S_local, N, D]; k, v [B, S_local, Nkv, D], sharded as ``usp_local_indices`` describes."""
    def inner(qq, kk, vv):
        if ring_group is None or dist.get_world_size(ring_group) == 1:
            return ops.attention_dense(qq, kk, vv, causal=causal, softmax_scale=softmax_scale)
        return ring_attention(qq, kk, vv, ring_group, causal=causal, softmax_scale=softmax_scale)
    return ulysses_attention(inner, q, k, v, ulysses_group)


class _HostParked:
    """A tensor kept in pinned host memory between uses (asynchronous copies on the current stream)."""

    def __init__(self, t: torch.Tensor, enabled: bool):
        self.enabled = enabled and t.is_cuda
        if self.enabled:
            self.host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            self.host.copy_(t, non_blocking=True)
            self.device = t.device
        else:
            self.t = t

    def get(self) -> torch.Tensor:
        return self.host.to(self.device, non_blocking=True) if self.enabled else self.t


def fpdt_attention(q, k, v, group, chunk: int, causal: bool = True, offload: bool = False,
                   softmax_scale: Optional[float] = None):
    """Chunked Ulysses attention.  Inputs are sequence-sharded contiguously: rank r holds [r*S_local, (r+1)*S_local).

    The local sequence is cut into chunks of ``chunk`` tokens.  For chunk index c every rank contributes its c-th
    local chunk, so after the all-to-all a rank holds (for its heads) the tokens {r*S_local + c*chunk + j}; the
    global order of gathered positions is therefore (rank, chunk, j).  Causal masking needs true positions, so the
    gathered K/V are kept in (chunk, rank, j) storage order together with their position vector, and each query
    chunk attends to all gathered keys with an explicit position comparison folded into a varlen call per rank
    segment.  Offloaded K/V chunks are parked in pinned host memory.
    """
    world = dist.get_world_size(group) if group is not None else 1
    B, S, N, D = q.shape
    if world == 1:
        return ops.attention_dense(q, k, v, causal=causal, softmax_scale=softmax_scale)
    if S % chunk:
        raise ValueError(f"local sequence {S} must be a multiple of chunk {chunk}")
    k, v = repeat_kv_for_ulysses(k, v, world)
    nc = S // chunk
    ks: List[_HostParked] = []
    vs: List[_HostParked] = []
    for c in range(nc):
        sl = slice(c * chunk, (c + 1) * chunk)
        # gathered layout along dim 1: [rank0 chunk c | rank1 chunk c | ...]
        ks.append(_HostParked(all_to_all(k[:, sl], group, scatter_dim=2, gather_dim=1), offload))
        vs.append(_HostParked(all_to_all(v[:, sl], group, scatter_dim=2, gather_dim=1), offload))
    outs = []
    for c in range(nc):
        sl = slice(c * chunk, (c + 1) * chunk)
        qc = all_to_all(q[:, sl], group, scatter_dim=2, gather_dim=1)            # [B, world*chunk, N/P, D]
        o_rows = []
        for r in range(world):                   # queries that came from rank r sit at true positions r*S + c*chunk + j
            qr = qc[:, r * chunk:(r + 1) * chunk]
            if not causal:
                kk = torch.cat([x.get() for x in ks], dim=1)
                vv = torch.cat([x.get() for x in vs], dim=1)
                o_rows.append(ops.attention_dense(qr, kk, vv, causal=False, softmax_scale=softmax_scale))
                continue
            # visible keys: every chunk of ranks < r, and chunks <= c of rank r (the last one causally)
            parts_k, parts_v = [], []
            for r2 in range(r):
                for c2 in range(nc):
                    parts_k.append(ks[c2].get()[:, r2 * chunk:(r2 + 1) * chunk])
                    parts_v.append(vs[c2].get()[:, r2 * chunk:(r2 + 1) * chunk])
            for c2 in range(c + 1):
                parts_k.append(ks[c2].get()[:, r * chunk:(r + 1) * chunk])
                parts_v.append(vs[c2].get()[:, r * chunk:(r + 1) * chunk])
            kk, vv = torch.cat(parts_k, dim=1), torch.cat(parts_v, dim=1)
            # keys are now in true position order and end exactly at the query chunk's last position, so the
            # bottom-right aligned causal mask is the right one
            o_rows.append(ops.attention_dense(qr, kk, vv, causal=True, softmax_scale=softmax_scale))
        oc = torch.cat(o_rows, dim=1)
        outs.append(all_to_all(oc, group, scatter_dim=1, gather_dim=2))
    return torch.cat(outs, dim=1)
