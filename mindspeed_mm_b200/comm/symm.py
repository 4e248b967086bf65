"""Symmetric-memory runtime and the engine's peer-to-peer collectives.

One arena per rank is allocated through ``torch.distributed._symmetric_memory`` (CUDA VMM allocation +
handle exchange), so every rank knows the address of every peer's arena and all arenas share one layout:

    [ flag block | gradient slot 0 | gradient slot 1 | bf16 parameter shards of every flat group ... ]

The kernels in ``ops/csrc/p2p.cu`` read peers' shards (all-gather) and peers' gradient slots
(reduce-scatter fused with the fp32 cast, the 1/N scale and the sharded AdamW update) with plain loads over
NVLink; nothing on this path calls NCCL.  The reference delegates the same two collectives to
``torch.distributed`` (HCCL/NCCL) inside FSDP2 (mindspeed_mm/fsdp/ops/fully_shard/fully_shard.py:481-825).

Host-side protocol per gradient publication (slot = unit parity, seq grows by one per use of the slot):
  compute stream: wait_done(slot, previous seq)  -> copy gradients into the slot
  comm stream   : rs kernel = publish ready[slot]=seq -> wait peers' ready -> reduce(+update) -> write done flags
``finish_step`` ends with a device-side barrier of the arena (``p2p_barrier_kernel``: sequence flags in the arena,
bounded wait, time-out reported through the status word), so a rank never gathers a shard that its owner has not
finished updating.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import native

ALIGN_BYTES = 1024


def _round_up(x, m):
    return (x + m - 1) // m * m


class SymmArena:
    """A byte arena that exists at the same offsets on every rank of ``group``."""

    def __init__(self, nbytes: int, group: dist.ProcessGroup, device: torch.device):
        import torch.distributed._symmetric_memory as symm
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.nbytes = _round_up(nbytes, ALIGN_BYTES) + ALIGN_BYTES       # + the barrier block carved below
        self.buf = symm.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buf, group)
        self.peer_base: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        if self.peer_base[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric memory: local base pointer mismatch")
        self.buf.zero_()
        self._cursor = 0
        # barrier block: one sequence flag per rank, written by the peers (see p2p_barrier_kernel)
        self._bar_off = self.carve(native.lib().mm_p2p_barrier_bytes())
        self._bar_ptrs = self.peer_ptrs(self._bar_off)
        self._bar_seq = 0

    def carve(self, nbytes: int) -> int:
        off = self._cursor
        self._cursor = _round_up(off + nbytes, ALIGN_BYTES)
        if self._cursor > self.nbytes:
            raise RuntimeError("symmetric arena exhausted")
        return off

    def view(self, off: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nb = numel * torch.empty(0, dtype=dtype).element_size()
        return self.buf[off:off + nb].view(dtype)

    def peer_ptrs(self, off: int):
        """ctypes array of every rank's address of arena offset ``off``."""
        arr = (C.c_void_p * self.world)(*[b + off for b in self.peer_base])
        return arr

    def barrier(self):
        """Stream-ordered barrier over the ranks of the arena, with a bounded device wait: a peer that never arrives
        makes the kernel write MM_TIMEOUT_PEER into the status word (``native.check_status`` raises on the host) and
        return; the context stays usable."""
        self._bar_seq += 1
        rc = native.lib().mm_p2p_barrier(self._bar_ptrs, self.world, self.rank, self._bar_seq,
                                         native.status_word(self.device).data_ptr(), native._st())
        native._check(rc, "p2p_barrier")

    def host_barrier(self):
        """Everything queued so far on this device is finished on every rank, and visible to the peers' kernels:
        device synchronize, process-group barrier, arena barrier.  Used after parameter loads that write the shards
        in the arena from the host side (no collective orders them against a peer's first gather)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.barrier()


class P2PCollectives:
    """Engine plug-in: moves the bf16 shards and the gradient slots into the arena and runs the kernels."""

    def __init__(self, engine, ag_ctas: int = 64, rs_ctas: int = 296, gather: Optional[str] = None):
        import os
        self.e = engine
        self.ag_ctas, self.rs_ctas = ag_ctas, rs_ctas
        # "ce": the parameter gather runs on the copy engines (one peer-to-peer async copy per shard): the parameters
        # are known a unit ahead, so the transfer needs no SM and the persistent GEMM keeps all of them.
        # "sm": the pull kernel (64 CTAs sharing SMs with the GEMM).
        self.gather = gather or os.environ.get("MM_B200_PARAM_GATHER", "ce")
        self.rs_ctas = int(os.environ.get("MM_B200_RS_CTAS", self.rs_ctas))
        groups = [g for u in engine.units for g in u.groups]
        flag_bytes = native.lib().mm_p2p_flag_bytes()
        slot_bytes = _round_up(max(g.padded for g in groups) * 2, ALIGN_BYTES)
        shard_bytes = sum(_round_up(g.shard_numel * 2, ALIGN_BYTES) for g in groups)
        total = _round_up(flag_bytes, ALIGN_BYTES) + 2 * slot_bytes + shard_bytes + 2 * ALIGN_BYTES
        self.arena = SymmArena(total, engine.group, engine.device)
        a = self.arena
        self.flag_off = a.carve(flag_bytes)
        self.slot_off = [a.carve(slot_bytes), a.carve(slot_bytes)]
        self.slot_elems = slot_bytes // 2
        self.flag_ptrs = a.peer_ptrs(self.flag_off)
        self.slot_ptrs = [a.peer_ptrs(self.slot_off[0]), a.peer_ptrs(self.slot_off[1])]
        self.slot_seq = [0, 0]
        self.shard_ptrs: Dict[int, object] = {}
        for g in groups:                      # re-home the persistent bf16 shards inside the arena
            off = a.carve(g.shard_numel * 2)
            new = a.view(off, g.shard_numel, torch.bfloat16)
            new.copy_(g.shard16)
            g.shard16 = new
            self.shard_ptrs[id(g)] = a.peer_ptrs(off)
        self._next_slot = 0
        a.host_barrier()

    # ------------------------------------------------------------------ all-gather
    def all_gather(self, g, full: torch.Tensor) -> None:
        if self.gather == "ce":
            rc = native.lib().mm_p2p_allgather_ce(self.shard_ptrs[id(g)], full.data_ptr(), g.shard_numel * 2, g.world,
                                                  g.rank, native._st())
        else:
            rc = native.lib().mm_p2p_allgather(self.shard_ptrs[id(g)], full.data_ptr(), g.shard_numel, g.world, g.rank,
                                               self.ag_ctas, native._st())
        native._check(rc, "p2p_allgather")

    # ------------------------------------------------------------------ gradient slots
    def grad_slot(self, g) -> torch.Tensor:
        """Next gradient slot as a flat bf16 tensor (compute stream waits until its last readers are done)."""
        s = self._next_slot
        self._next_slot ^= 1
        if self.slot_seq[s] > 0:
            rc = native.lib().mm_p2p_wait_done(self.arena.peer_base[g.rank] + self.flag_off, s, self.slot_seq[s],
                                               g.world, g.rank, native.status_word(self.e.device).data_ptr(),
                                               native._st())
            native._check(rc, "p2p_wait_done")
        g._slot = s
        return self.arena.view(self.slot_off[s], g.padded, torch.bfloat16)

    def reduce_scatter_update(self, g, flat: torch.Tensor, fused: bool, engine) -> None:
        s = g._slot
        self.slot_seq[s] += 1
        seq = self.slot_seq[s]
        st = native.status_word(engine.device).data_ptr()
        inv = 1.0 / engine.grad_divide
        L = native.lib()
        if fused:
            g.step_count += 1
            o = engine.opt
            split = min(max(g.decay_end - g.rank * g.shard_numel, 0), g.shard_numel)
            rc = L.mm_p2p_rs_adamw(self.slot_ptrs[s], self.flag_ptrs, g.shard_numel, g.world, g.rank, s, seq, inv,
                                   g.master.data_ptr(), g.exp_avg.data_ptr(), g.exp_avg_sq.data_ptr(),
                                   g.shard16.data_ptr(), split, engine.lr * g.lr_scale, o.betas[0], o.betas[1], o.eps,
                                   o.weight_decay, 1.0 - o.betas[0] ** g.step_count, 1.0 - o.betas[1] ** g.step_count,
                                   st, self.rs_ctas, native._st())
            native._check(rc, "p2p_rs_adamw")
        else:
            acc = g.grad32 is not None
            if not acc:
                g.grad32 = torch.empty(g.shard_numel, dtype=torch.float32, device=engine.device)
            rc = L.mm_p2p_rs(self.slot_ptrs[s], self.flag_ptrs, g.shard_numel, g.world, g.rank, s, seq, inv,
                             g.grad32.data_ptr(), int(acc), st, self.rs_ctas, native._st())
            native._check(rc, "p2p_rs")

    def step_barrier(self):
        self.arena.barrier()

    def sync_after_load(self):
        self.arena.host_barrier()

