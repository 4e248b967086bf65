"""GEMMs whose epilogue IS the collective (outputs are written into peers' symmetric buffers over NVLink).

* ``UlyssesQKVProjection``  - y = x W_qkv^T + b on this rank's sequence slice; every 64-column output slab is
  stored straight into the rank that owns those heads, at this rank's row offset of the full sequence.  After a
  barrier each rank holds q|k|v for ITS heads over the FULL sequence: the three all-to-alls of Ulysses
  (mindspeed_mm/fsdp/ops/flash_attn/flash_attn.py:439-461, fsdp/models/wan2_2/modeling_wan2_2.py:389-394) never run as
  separate collectives.
* ``RowParallelLinearRS``   - tensor-parallel row-parallel linear followed by a reduce-scatter over the sequence
  (Megatron sequence parallelism): every rank pushes its partial 128-row tiles into a per-source slot on the row
  block's owner, which folds the slots (fp32 accumulate).  Replaces GEMM -> NCCL reduce-scatter.
Backward passes use the plain collectives (all-to-all / all-gather over NCCL) followed by the tcgen05 dgrad / wgrad
GEMMs.  Both modules own a symmetric buffer sized at construction; ``forward`` brackets the kernel with the
device-side barrier of the arena (stream ordered, no host sync).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native
from .symm import SymmArena


def _declare():
    L = native.lib()
    p, i, ll = C.c_void_p, C.c_int, C.c_longlong
    L.mm_gemm_bf16_routed.argtypes = [p, p, p, i, i, i, ll, ll, p, ll, ll, ll, i, i, i, i, i, p, p]
    L.mm_gemm_bf16_routed.restype = i
    L.mm_fold_slots.argtypes = [p, p, ll, i, ll, i, p]
    L.mm_fold_slots.restype = i
    return L


class _UlyssesQKVFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, mod):
        L = _declare()
        S_local, H = x.shape
        N = w.shape[0]
        a = mod.arena
        a.barrier()                                   # everyone is done reading the previous contents of recv
        rc = L.mm_gemm_bf16_routed(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(), S_local, N, H,
                                   x.stride(0), w.stride(0), mod.recv_ptrs, mod.S_full, mod.cols, mod.cols, 1, mod.blk,
                                   mod.world, mod.rank, mod.rank * S_local, native.status_word(x.device).data_ptr(),
                                   native._st())
        native._check(rc, "gemm_routed(ulysses)")
        a.barrier()                                   # all slabs from all peers have landed
        ctx.save_for_backward(x, w)
        ctx.mod, ctx.has_bias = mod, bias is not None
        return mod.recv.clone()

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        mod = ctx.mod
        W, blk, S_local = mod.world, mod.blk, x.shape[0]
        # g: [S_full, n_slots * blk] for my head group -> all-to-all back to [S_local, N] in the original column order
        n_slots = mod.cols // blk
        send = g.view(W, S_local, n_slots, blk).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=mod.group)        # recv[src] = grad of my rows for src's head group
        dy = recv.permute(1, 2, 0, 3).reshape(S_local, n_slots * W * blk)   # column = (slot * W + dst) * blk + c
        dx = native.gemm_nn(dy, w)
        dw = native.gemm_tn(dy, x)
        db = torch.sum(dy, 0, dtype=torch.float32).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db, None


class UlyssesQKVProjection:
    """``q, k, v = proj(x_local)`` with x_local [S_local, H] (equal slices on every rank) and W [n_slots*H_out, H];
    returns [S_full, n_slots * H_out / world] = the q|k|v slots of this rank's heads."""

    def __init__(self, group, device, S_local: int, out_features: int, n_slots: int = 3):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        per_slot = out_features // n_slots
        if per_slot % self.world or (per_slot // self.world) % 64:
            raise ValueError("per-rank head block must be a multiple of 64 columns")
        self.blk = per_slot // self.world
        self.cols = n_slots * self.blk
        self.S_full = S_local * self.world
        self.arena = SymmArena(self.S_full * self.cols * 2 + 4096, group, torch.device(device))
        off = self.arena.carve(self.S_full * self.cols * 2)
        self.recv = self.arena.view(off, self.S_full * self.cols, torch.bfloat16).view(self.S_full, self.cols)
        self.recv_ptrs = self.arena.peer_ptrs(off)

    def __call__(self, x, w, bias=None):
        return _UlyssesQKVFn.apply(x.contiguous(), w, bias, self)


class _RowParallelRSFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, mod):
        L = _declare()
        M, K = x.shape
        N = w.shape[0]
        a = mod.arena
        a.barrier()
        rc = L.mm_gemm_bf16_routed(x.data_ptr(), w.data_ptr(), None, M, N, K, x.stride(0), w.stride(0), mod.slot_ptrs,
                                   M, N, N, 2, mod.rows, mod.world, mod.rank, 0,
                                   native.status_word(x.device).data_ptr(), native._st())
        native._check(rc, "gemm_routed(rs)")
        a.barrier()
        out = torch.empty(mod.rows, N, dtype=x.dtype, device=x.device)
        native._check(L.mm_fold_slots(mod.slots.data_ptr(), out.data_ptr(), mod.rows, N, N, mod.world, native._st()),
                      "fold_slots")
        ctx.save_for_backward(x, w)
        ctx.mod = mod
        return out

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        mod = ctx.mod
        outs = torch.empty(mod.world * g.shape[0], g.shape[1], dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(outs, g.contiguous(), group=mod.group)
        return native.gemm_nn(outs, w), native.gemm_tn(outs, x), None


class RowParallelLinearRS:
    """``y_local = reduce_scatter_rows(x @ W_local^T)``: x [M, K/tp], W_local [N, K/tp] -> [M/tp, N]."""

    def __init__(self, group, device, M: int, N: int):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if M % self.world or (M // self.world) % 128:
            raise ValueError("rows per rank must be a multiple of 128")
        self.rows = M // self.world
        self.arena = SymmArena(M * N * 2 + 4096, group, torch.device(device))
        off = self.arena.carve(M * N * 2)
        self.slots = self.arena.view(off, M * N, torch.bfloat16).view(M, N)     # [world (source) * rows, N]
        self.slot_ptrs = self.arena.peer_ptrs(off)

    def __call__(self, x, w):
        return _RowParallelRSFn.apply(x.contiguous(), w, self)


# ------------------------------------------------------------------------------------------ gather -> GEMM
def _declare_gather():
    L = native.lib()
    p, i, ll, u = C.c_void_p, C.c_int, C.c_longlong, C.c_uint
    L.mm_gemm_gather_bf16.argtypes = [p, p, p, p, i, i, i, ll, ll, ll, p, ll, i, i, i, i, i, i, p, u, p, p]
    L.mm_gemm_gather_bf16.restype = i
    return L


class _GatherGemmBase:
    def _launch(self, A, w, bias, out, src_ptrs, src_pitch, src_rows, src_cols, axis, extent):
        L = _declare_gather()
        self.epoch += 1
        M, K = A.shape
        rc = L.mm_gemm_gather_bf16(A.data_ptr(), w.data_ptr(), out.data_ptr(), None if bias is None else bias.data_ptr(),
                                   M, w.shape[0], K, A.stride(0), w.stride(0), out.stride(0), src_ptrs, src_pitch, src_rows,
                                   src_cols, axis, extent, self.world, self.rank, self.flags.data_ptr(), self.epoch,
                                   native.status_word(A.device).data_ptr(), native._st())
        native._check(rc, "gemm_gather")


class _AllGatherLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, mod):
        S_local, H = x.shape
        mod.send.copy_(x)                                       # peers read my slab from here
        mod.A[mod.rank * S_local:(mod.rank + 1) * S_local].copy_(x)
        out = torch.empty(mod.A.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        mod.arena.barrier()                                     # every rank's send buffer is written
        mod._launch(mod.A, w, bias, out, mod.send_ptrs, H, S_local, H, 0, S_local)
        mod.arena.barrier()                                     # every rank is done reading my send buffer
        ctx.save_for_backward(mod.A.clone(), w)
        ctx.mod, ctx.has_bias = mod, bias is not None
        return out

    @staticmethod
    def backward(ctx, g):
        A, w = ctx.saved_tensors
        mod = ctx.mod
        dA = native.gemm_nn(g.contiguous(), w)
        dx = torch.empty(A.shape[0] // mod.world, A.shape[1], dtype=dA.dtype, device=dA.device)
        dist.reduce_scatter_tensor(dx, dA, group=mod.group)
        db = torch.sum(g, 0, dtype=torch.float32).to(g.dtype) if ctx.has_bias else None
        return dx, native.gemm_tn(g.contiguous(), A), db, None


class AllGatherLinear(_GatherGemmBase):
    """Sequence-parallel all-gather fused into a column-parallel linear:
    ``y = all_gather_rows(x_local) @ W_local^T (+ b)``, x_local [S/tp, H] (S/tp a multiple of 128) -> y [S, N/tp]."""

    def __init__(self, group, device, S_local: int, H: int):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if S_local % 128:
            raise ValueError("rows per rank must be a multiple of 128")
        self.arena = SymmArena(S_local * H * 2 + 4096, group, torch.device(device))
        off = self.arena.carve(S_local * H * 2)
        self.send = self.arena.view(off, S_local * H, torch.bfloat16).view(S_local, H)
        self.send_ptrs = self.arena.peer_ptrs(off)
        self.A = torch.empty(S_local * self.world, H, dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(8, dtype=torch.int32, device=device)
        self.epoch = 0

    def __call__(self, x, w, bias=None):
        return _AllGatherLinearFn.apply(x.contiguous(), w, bias, self)


class _UlyssesOutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o_heads, w, bias, mod):
        S_full, cols = o_heads.shape
        S_local = S_full // mod.world
        mod.o_buf.copy_(o_heads)
        mod.A[:, mod.rank * cols:(mod.rank + 1) * cols].copy_(o_heads[mod.rank * S_local:(mod.rank + 1) * S_local])
        out = torch.empty(S_local, w.shape[0], dtype=o_heads.dtype, device=o_heads.device)
        mod.arena.barrier()
        mod._launch(mod.A, w, bias, out, mod.src_ptrs, cols, S_local, cols, 2, cols)
        mod.arena.barrier()
        ctx.save_for_backward(mod.A.clone(), w)
        ctx.mod, ctx.has_bias = mod, bias is not None
        return out

    @staticmethod
    def backward(ctx, g):
        A, w = ctx.saved_tensors
        mod = ctx.mod
        S_local, H = A.shape
        cols = H // mod.world
        dA = native.gemm_nn(g.contiguous(), w)                                  # [S_local, H]
        send = dA.view(S_local, mod.world, cols).permute(1, 0, 2).contiguous()  # [dst head group, S_local, cols]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=mod.group)                     # [src rows block, S_local, cols]
        db = torch.sum(g, 0, dtype=torch.float32).to(g.dtype) if ctx.has_bias else None
        return recv.reshape(mod.world * S_local, cols), native.gemm_tn(g.contiguous(), A), db, None


class UlyssesOutProjection(_GatherGemmBase):
    """Ulysses output projection with the head all-to-all fused into the GEMM's operand fetch:
    o_heads [S_full, H/P] (this rank's heads, all tokens) -> y [S_local, N] = concat_heads(o)[my tokens] @ W^T (+ b)."""

    def __init__(self, group, device, S_local: int, H: int):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        cols = H // self.world
        if cols % 64:
            raise ValueError("per-rank head block must be a multiple of 64 columns")
        S_full = S_local * self.world
        self.arena = SymmArena(S_full * cols * 2 + 4096, group, torch.device(device))
        off = self.arena.carve(S_full * cols * 2)
        self.o_buf = self.arena.view(off, S_full * cols, torch.bfloat16).view(S_full, cols)
        # every peer reads the rows of MY tokens out of ITS buffer: same offset on every peer
        row_off = self.rank * S_local * cols * 2
        self.src_ptrs = (C.c_void_p * self.world)(*[b + off + row_off for b in self.arena.peer_base])
        self.A = torch.empty(S_local, H, dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(8, dtype=torch.int32, device=device)
        self.epoch = 0

    def __call__(self, o_heads, w, bias=None):
        return _UlyssesOutFn.apply(o_heads.contiguous(), w, bias, self)
