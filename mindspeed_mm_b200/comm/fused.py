"""GEMMs whose prologue or epilogue IS the collective, forward and backward, over NVLink peer memory.

Four linear layers, each a pair of tcgen05 kernels (``ops/csrc/gemm.cu`` routed epilogue, ``ops/csrc/gemm_gather.cu``
gathering producer).  The backward of a layer whose forward scatters is a gather and the other way round, so every
pass below is one of those two kernels; nothing on these paths calls NCCL.

==========================  ===================================  ====================================================
layer                       forward                              backward (data gradient; weight gradient is local)
==========================  ===================================  ====================================================
``AllGatherLinear``         rows gathered inside the GEMM        dA = g W pushed as row blocks into per-source slots
(sequence-parallel column)  (gather, axis 0)                     on the row owner, folded there (routed, mode 2)
``RowParallelLinearRS``     partial rows pushed into slots on    rows of g gathered inside dx = gather(g) W
(sequence-parallel row)     the row owner (routed, mode 2)       (gather, axis 0)
``UlyssesQKVProjection``    head blocks stored into the head     my rows' gradient comes back from every head owner
                            owner's buffer (routed, mode 1)      inside dx = gather(g) W' (gather, axis 2)
``UlyssesOutProjection``    heads fetched from their owners      dA = g W stored as head blocks into the head owners
                            inside the GEMM (gather, axis 2)     (routed, mode 1)
==========================  ===================================  ====================================================

The reference runs these as separate collectives around library GEMMs: Megatron column / row parallel linears
(mindspeed_mm/models/common/attention.py:296-389) and Ulysses all-to-alls around the attention core
(mindspeed_mm/fsdp/ops/flash_attn/flash_attn.py:439-461, fsdp/models/wan2_2/modeling_wan2_2.py:389-394).

Every module owns symmetric buffers sized at construction and brackets its kernels with the arena's bounded
device-side barrier (stream ordered, no host sync).  Modules are shared by all layers of the same shape
(``shared``): calls are issued on one stream, and autograd never keeps a view of a shared buffer.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import native
from .symm import SymmArena

_DECLARED = False


def _lib():
    global _DECLARED
    L = native.lib()
    if not _DECLARED:
        p, i, ll, u = C.c_void_p, C.c_int, C.c_longlong, C.c_uint
        L.mm_gemm_bf16_routed_ex.argtypes = [p, p, p, i, i, i, ll, ll, p, ll, ll, ll, i, i, i, i, i, i, p, p]
        L.mm_gemm_bf16_routed_ex.restype = i
        L.mm_gemm_bf16_routed_stats.argtypes = [p, p, p, i, i, i, ll, ll, p, ll, ll, ll, i, i, i, i, p, i, p, p]
        L.mm_gemm_bf16_routed_stats.restype = i
        L.mm_fold_slots.argtypes = [p, p, ll, i, ll, i, p]
        L.mm_fold_slots.restype = i
        L.mm_gemm_gather_bf16_ex.argtypes = [p, p, p, p, i, i, i, ll, ll, ll, p, ll, i, i, i, i, i, i, p, u, i, p, p]
        L.mm_gemm_gather_bf16_ex.restype = i
        _DECLARED = True
    return L


def _routed(x, w, bias, M, N, K, ldb, dst_ptrs, dst_rows, dst_cols, ldc, mode, blk, world, rank, row_off, b_mn, what):
    """``x [M, K] (*) w`` with the output tiles stored into ``dst_ptrs`` (see ``mm_gemm_bf16_routed_ex``)."""
    rc = _lib().mm_gemm_bf16_routed_ex(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(), M, N, K,
                                       x.stride(0), ldb, dst_ptrs, dst_rows, dst_cols, ldc, mode, blk, world, rank,
                                       row_off, int(b_mn), native.status_word(x.device).data_ptr(), native._st())
    native._check(rc, what)


class _Gatherer:
    """State of one use of the gathering GEMM: its arrival counters count up by one grid per launch, so every
    (buffer, GEMM shape) pair keeps its own counters and epoch."""

    def __init__(self, device):
        self.flags = torch.zeros(8, dtype=torch.int32, device=device)
        self.epoch = 0

    def launch(self, A, w, bias, out, src_ptrs, src_pitch, src_rows, src_cols, axis, extent, world, rank, b_mn, what):
        self.epoch += 1
        M, K = A.shape
        N = out.shape[1]
        rc = _lib().mm_gemm_gather_bf16_ex(A.data_ptr(), w.data_ptr(), out.data_ptr(),
                                           None if bias is None else bias.data_ptr(), M, N, K, A.stride(0), w.stride(0),
                                           out.stride(0), src_ptrs, src_pitch, src_rows, src_cols, axis, extent, world,
                                           rank, self.flags.data_ptr(), self.epoch, int(b_mn),
                                           native.status_word(A.device).data_ptr(), native._st())
        native._check(rc, what)


_SHARED: Dict[Tuple, object] = {}


def shared(cls, group, device, *shape):
    """One module per (class, group, shape): layers of equal shape reuse its symmetric buffers."""
    key = (cls.__name__, id(group), str(device), shape)
    if key not in _SHARED:
        _SHARED[key] = cls(group, device, *shape)
    return _SHARED[key]


def fused_supported(x: torch.Tensor) -> bool:
    from .. import ops
    return x.is_cuda and x.dtype == torch.bfloat16 and ops.get_tier() == "native"


# ------------------------------------------------------------------------------------------ sequence-parallel column linear
class _AllGatherLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, mod):
        S_local, H = x.shape
        mod.send.copy_(x)                                       # peers read my slab from here
        mod.A[mod.rank * S_local:(mod.rank + 1) * S_local].copy_(x)
        out = torch.empty(mod.A.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        mod.arena.barrier()                                     # every rank's send buffer is written
        mod.fwd.launch(mod.A, w, bias, out, mod.send_ptrs, H, S_local, H, 0, S_local, mod.world, mod.rank, 0,
                       "gemm_gather(allgather_linear)")
        mod.arena.barrier()                                     # every rank is done reading my send buffer
        ctx.save_for_backward(mod.A.clone(), w)
        ctx.mod, ctx.has_bias = mod, bias is not None
        return out

    @staticmethod
    def backward(ctx, g):
        A, w = ctx.saved_tensors
        mod = ctx.mod
        g = g.contiguous()
        S, H = A.shape
        # dA = g W (NN); its row block r belongs to rank r: pushed into my slot of r's buffer, folded by r
        mod.arena.barrier()                                     # the slots' previous contents have been folded
        _routed(g, w, None, S, H, g.shape[1], w.stride(0), mod.slot_ptrs, S, H, H, 2, mod.rows, mod.world, mod.rank, 0,
                True, "gemm_routed(allgather_linear dgrad)")
        mod.arena.barrier()                                     # all partial row blocks have landed
        dx = torch.empty(mod.rows, H, dtype=g.dtype, device=g.device)
        native._check(_lib().mm_fold_slots(mod.slots.data_ptr(), dx.data_ptr(), mod.rows, H, H, mod.world, native._st()),
                      "fold_slots")
        db = torch.sum(g, 0, dtype=torch.float32).to(g.dtype) if ctx.has_bias else None
        return dx, native.gemm_tn(g, A), db, None


class AllGatherLinear:
    """Sequence-parallel all-gather fused into a column-parallel linear:
    ``y = all_gather_rows(x_local) @ W_local^T (+ b)``, x_local [S/tp, H] (S/tp a multiple of 128) -> y [S, N/tp]."""

    def __init__(self, group, device, S_local: int, H: int):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if S_local % 128 or H % 64:
            raise ValueError("rows per rank must be a multiple of 128 and the hidden size a multiple of 64")
        self.rows = S_local
        S = S_local * self.world
        self.arena = SymmArena((S_local + S) * H * 2 + 8192, group, torch.device(device))
        off = self.arena.carve(S_local * H * 2)
        self.send = self.arena.view(off, S_local * H, torch.bfloat16).view(S_local, H)
        self.send_ptrs = self.arena.peer_ptrs(off)
        off = self.arena.carve(S * H * 2)                       # backward: [source rank, my rows, H]
        self.slots = self.arena.view(off, S * H, torch.bfloat16).view(S, H)
        self.slot_ptrs = self.arena.peer_ptrs(off)
        self.A = torch.empty(S, H, dtype=torch.bfloat16, device=device)
        self.fwd = _Gatherer(device)

    def __call__(self, x, w, bias=None):
        return _AllGatherLinearFn.apply(x.contiguous(), w, bias, self)


# ------------------------------------------------------------------------------------------ sequence-parallel row linear
class _RowParallelRSFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, mod):
        M, K = x.shape
        N = w.shape[0]
        mod.arena.barrier()
        _routed(x, w, None, M, N, K, w.stride(0), mod.slot_ptrs, M, N, N, 2, mod.rows, mod.world, mod.rank, 0, False,
                "gemm_routed(rs)")
        mod.arena.barrier()
        out = torch.empty(mod.rows, N, dtype=x.dtype, device=x.device)
        native._check(_lib().mm_fold_slots(mod.slots.data_ptr(), out.data_ptr(), mod.rows, N, N, mod.world, native._st()),
                      "fold_slots")
        ctx.save_for_backward(x, w)
        ctx.mod = mod
        return out

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        mod = ctx.mod
        M, K = x.shape
        N = w.shape[0]
        mod.send.copy_(g)
        mod.G[mod.rank * mod.rows:(mod.rank + 1) * mod.rows].copy_(g)
        dx = torch.empty(M, K, dtype=x.dtype, device=x.device)
        mod.arena.barrier()                                     # every rank's gradient rows are in its send buffer
        # dx = gather_rows(g) W (NN): the row blocks of g arrive from their owners while the GEMM runs
        mod.bwd.launch(mod.G, w, None, dx, mod.send_ptrs, N, mod.rows, N, 0, mod.rows, mod.world, mod.rank, 1,
                       "gemm_gather(rs dgrad)")
        mod.arena.barrier()
        return dx, native.gemm_tn(mod.G, x), None


class RowParallelLinearRS:
    """``y_local = reduce_scatter_rows(x @ W_local^T)``: x [M, K/tp], W_local [N, K/tp] -> [M/tp, N]."""

    def __init__(self, group, device, M: int, N: int):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if M % self.world or (M // self.world) % 128 or N % 64:
            raise ValueError("rows per rank must be a multiple of 128 and the output width a multiple of 64")
        self.rows = M // self.world
        self.arena = SymmArena((M + self.rows) * N * 2 + 8192, group, torch.device(device))
        off = self.arena.carve(M * N * 2)
        self.slots = self.arena.view(off, M * N, torch.bfloat16).view(M, N)     # [world (source) * rows, N]
        self.slot_ptrs = self.arena.peer_ptrs(off)
        off = self.arena.carve(self.rows * N * 2)               # backward: my gradient rows, read by every peer
        self.send = self.arena.view(off, self.rows * N, torch.bfloat16).view(self.rows, N)
        self.send_ptrs = self.arena.peer_ptrs(off)
        self.G = torch.empty(M, N, dtype=torch.bfloat16, device=device)
        self.bwd = _Gatherer(device)

    def __call__(self, x, w):
        return _RowParallelRSFn.apply(x.contiguous(), w, self)


# ------------------------------------------------------------------------------------------ Ulysses: QKV projection
def _to_owner_major(t: torch.Tensor, world: int, n_slots: int, blk: int) -> torch.Tensor:
    """Rows (or entries) ordered (slot, owner, c) -> (owner, slot, c): the order in which the gathered gradient holds
    its columns (one contiguous block per head owner)."""
    return t.view(n_slots, world, blk, *t.shape[1:]).transpose(0, 1).reshape(t.shape)


def _from_owner_major(t: torch.Tensor, world: int, n_slots: int, blk: int) -> torch.Tensor:
    return t.view(world, n_slots, blk, *t.shape[1:]).transpose(0, 1).reshape(t.shape)


class _UlyssesQKVFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, mod):
        S_local, H = x.shape
        N = w.shape[0]
        a = mod.arena
        a.barrier()                                   # everyone is done reading the previous contents of recv
        if mod.with_stats:
            mod.stats_local.zero_()
            rc = _lib().mm_gemm_bf16_routed_stats(x.data_ptr(), w.data_ptr(), None if bias is None else bias.data_ptr(),
                                                  S_local, N, H, x.stride(0), w.stride(0), mod.recv_ptrs, mod.S_full,
                                                  mod.cols, mod.cols, mod.blk, mod.world, mod.rank, mod.rank * S_local,
                                                  mod.stats_local.data_ptr(), mod.n_slots,
                                                  native.status_word(x.device).data_ptr(), native._st())
            native._check(rc, "gemm_routed(ulysses+stats)")
            nb = mod.stats_local.numel() * 4          # rows padded to a multiple of 4: a 16-byte multiple per rank
            for p in range(mod.world):                # my rows' sums of squares go to every rank (a few KB each)
                native._check(native.lib().mm_p2p_copy(mod.stats_peer[p] + mod.rank * nb, mod.stats_local.data_ptr(), nb, 4,
                                                       native._st()), "p2p_copy(stats)")
        else:
            _routed(x, w, bias, S_local, N, H, w.stride(0), mod.recv_ptrs, mod.S_full, mod.cols, mod.cols, 1, mod.blk,
                    mod.world, mod.rank, mod.rank * S_local, False, "gemm_routed(ulysses)")
        a.barrier()                                   # all slabs from all peers have landed
        ctx.save_for_backward(x, w)
        ctx.mod, ctx.has_bias = mod, bias is not None
        out = mod.recv.clone()
        if mod.with_stats:
            stats = mod.stats_full[:, :S_local].reshape(mod.S_full, mod.n_slots)      # drops the row padding (copies)
            ctx.mark_non_differentiable(stats)
            return out, stats
        return out

    @staticmethod
    def backward(ctx, g, *_):
        x, w = ctx.saved_tensors
        mod = ctx.mod
        W, blk, ns, cols = mod.world, mod.blk, mod.n_slots, mod.cols
        S_local, H = x.shape
        N = w.shape[0]
        # g: gradient of my heads' q|k|v over ALL rows.  Row block r of it belongs to rank r: every rank fetches its
        # rows from every head owner inside the data-gradient GEMM (K axis = (owner, slot, c)).
        mod.gbuf.copy_(g)
        mod.dY[:, mod.rank * cols:(mod.rank + 1) * cols].copy_(g[mod.rank * S_local:(mod.rank + 1) * S_local])
        w_om = _to_owner_major(w, W, ns, blk).contiguous()
        dx = torch.empty(S_local, H, dtype=x.dtype, device=x.device)
        mod.arena.barrier()                           # every head owner's gradient is in its gbuf
        mod.bwd.launch(mod.dY, w_om, None, dx, mod.g_src_ptrs, cols, S_local, cols, 2, cols, W, mod.rank, 1,
                       "gemm_gather(ulysses qkv dgrad)")
        mod.arena.barrier()                           # every rank is done reading my gbuf
        dw = _from_owner_major(native.gemm_tn(mod.dY, x), W, ns, blk)
        db = None
        if ctx.has_bias:
            db = _from_owner_major(torch.sum(mod.dY, 0, dtype=torch.float32).to(g.dtype), W, ns, blk)
        return dx, dw, db, None


class UlyssesQKVProjection:
    """``q, k, v = proj(x_local)`` with x_local [S_local, H] (equal slices on every rank) and W [n_slots*H_out, H];
    returns [S_full, n_slots * H_out / world] = the q|k|v slots of this rank's heads.  ``with_stats``: also returns
    [S_full, n_slots] fp32 = the sum of squares of every slot's FULL output row (all heads, taken from the GEMM's
    accumulators), which a normalisation over the whole hidden vector needs after the heads have been scattered."""

    def __init__(self, group, device, S_local: int, out_features: int, n_slots: int = 3, with_stats: bool = False):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        per_slot = out_features // n_slots
        if per_slot % self.world or (per_slot // self.world) % 64:
            raise ValueError("per-rank head block must be a multiple of 64 columns")
        self.n_slots, self.with_stats = n_slots, with_stats
        self.blk = per_slot // self.world
        self.cols = n_slots * self.blk
        self.S_full = S_local * self.world
        dev = torch.device(device)
        S_pad = (S_local + 3) // 4 * 4
        stat_bytes = self.world * S_pad * n_slots * 4
        self.arena = SymmArena(2 * self.S_full * self.cols * 2 + stat_bytes + 16384, group, dev)
        off = self.arena.carve(self.S_full * self.cols * 2)
        self.recv = self.arena.view(off, self.S_full * self.cols, torch.bfloat16).view(self.S_full, self.cols)
        self.recv_ptrs = self.arena.peer_ptrs(off)
        off = self.arena.carve(self.S_full * self.cols * 2)     # backward: my heads' gradient, read row-block-wise by peers
        self.gbuf = self.arena.view(off, self.S_full * self.cols, torch.bfloat16).view(self.S_full, self.cols)
        row_off = self.rank * S_local * self.cols * 2            # every peer serves the rows of MY tokens
        self.g_src_ptrs = (C.c_void_p * self.world)(*[b + off + row_off for b in self.arena.peer_base])
        off = self.arena.carve(stat_bytes)
        self.stats_full = self.arena.view(off, self.world * S_pad * n_slots, torch.float32).view(self.world, S_pad, n_slots)
        self.stats_peer = [b + off for b in self.arena.peer_base]
        self.stats_local = torch.zeros(S_pad, n_slots, dtype=torch.float32, device=dev)
        self.dY = torch.empty(S_local, self.world * self.cols, dtype=torch.bfloat16, device=dev)
        self.bwd = _Gatherer(dev)

    def __call__(self, x, w, bias=None):
        return _UlyssesQKVFn.apply(x.contiguous(), w, bias, self)


# ------------------------------------------------------------------------------------------ Ulysses: output projection
class _UlyssesOutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o_heads, w, bias, mod):
        S_full, cols = o_heads.shape
        S_local = S_full // mod.world
        mod.o_buf.copy_(o_heads)
        mod.A[:, mod.rank * cols:(mod.rank + 1) * cols].copy_(o_heads[mod.rank * S_local:(mod.rank + 1) * S_local])
        out = torch.empty(S_local, w.shape[0], dtype=o_heads.dtype, device=o_heads.device)
        mod.arena.barrier()
        mod.fwd.launch(mod.A, w, bias, out, mod.src_ptrs, cols, S_local, cols, 2, cols, mod.world, mod.rank, 0,
                       "gemm_gather(ulysses out)")
        mod.arena.barrier()
        ctx.save_for_backward(mod.A.clone(), w)
        ctx.mod, ctx.has_bias = mod, bias is not None
        return out

    @staticmethod
    def backward(ctx, g):
        A, w = ctx.saved_tensors
        mod = ctx.mod
        g = g.contiguous()
        S_local, H = A.shape
        cols = H // mod.world
        # dA = g W (NN) [S_local, H]; its column block c is the gradient of rank c's heads for my rows: stored straight
        # into rank c's buffer at my row offset
        mod.arena.barrier()                           # the previous contents of gbuf have been consumed
        _routed(g, w, None, S_local, H, g.shape[1], w.stride(0), mod.g_ptrs, S_local * mod.world, cols, cols, 1, cols,
                mod.world, mod.rank, mod.rank * S_local, True, "gemm_routed(ulysses out dgrad)")
        mod.arena.barrier()                           # every rank's block has landed
        db = torch.sum(g, 0, dtype=torch.float32).to(g.dtype) if ctx.has_bias else None
        return mod.gbuf.clone(), native.gemm_tn(g, A), db, None


class UlyssesOutProjection:
    """Ulysses output projection with the head all-to-all fused into the GEMM's operand fetch:
    o_heads [S_full, H/P] (this rank's heads, all tokens) -> y [S_local, N] = concat_heads(o)[my tokens] @ W^T (+ b)."""

    def __init__(self, group, device, S_local: int, H: int):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        cols = H // self.world
        if cols % 64:
            raise ValueError("per-rank head block must be a multiple of 64 columns")
        S_full = S_local * self.world
        self.arena = SymmArena(2 * S_full * cols * 2 + 8192, group, torch.device(device))
        off = self.arena.carve(S_full * cols * 2)
        self.o_buf = self.arena.view(off, S_full * cols, torch.bfloat16).view(S_full, cols)
        # every peer reads the rows of MY tokens out of ITS buffer: same offset on every peer
        row_off = self.rank * S_local * cols * 2
        self.src_ptrs = (C.c_void_p * self.world)(*[b + off + row_off for b in self.arena.peer_base])
        off = self.arena.carve(S_full * cols * 2)               # backward: gradient of my heads, written by every rank
        self.gbuf = self.arena.view(off, S_full * cols, torch.bfloat16).view(S_full, cols)
        self.g_ptrs = self.arena.peer_ptrs(off)
        self.A = torch.empty(S_local, H, dtype=torch.bfloat16, device=device)
        self.fwd = _Gatherer(device)

    def __call__(self, o_heads, w, bias=None):
        return _UlyssesOutFn.apply(o_heads.contiguous(), w, bias, self)


# ------------------------------------------------------------------------------------------ Ulysses: whole-row q/k norm + RoPE
def _declare_qk():
    L = native.lib()
    if not getattr(L, "_mm_qk_declared", False):
        p, i, ll, f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        L.mm_qk_norm_rope_fwd.argtypes = [p, ll, p, i, p, p, p, p, i, i, i, i, f, p]
        L.mm_qk_norm_rope_bwd_partials.argtypes = [p, ll, p, i, p, p, p, p, p, p, i, i, i, i, f, p]
        L.mm_qk_norm_rope_bwd.argtypes = [p, ll, p, i, p, p, p, p, p, i, p, ll, i, i, i, i, f, p]
        for fn in (L.mm_qk_norm_rope_fwd, L.mm_qk_norm_rope_bwd_partials, L.mm_qk_norm_rope_bwd):
            fn.restype = i
        L._mm_qk_declared = True
    return L


class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, raw, stats, wq, wk, cos, sin, mod):
        L = _declare_qk()
        T, blk, D = raw.shape[0], mod.blk, mod.D
        lo = mod.rank * blk
        w = torch.stack([wq[lo:lo + blk], wk[lo:lo + blk]]).to(torch.bfloat16).contiguous()      # my heads' channels
        out = torch.empty(2, T, blk, dtype=raw.dtype, device=raw.device)
        rc = L.mm_qk_norm_rope_fwd(raw.data_ptr(), raw.stride(0), stats.data_ptr(), stats.shape[1], w.data_ptr(),
                                   cos.data_ptr(), sin.data_ptr(), out.data_ptr(), T, blk, D, mod.H, mod.eps, native._st())
        native._check(rc, "qk_norm_rope_fwd")
        ctx.save_for_backward(raw, stats, w, cos, sin)
        ctx.mod = mod
        nh = blk // D
        return out[0].view(T, nh, D), out[1].view(T, nh, D), raw[:, 2 * blk:3 * blk].view(T, nh, D)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        L = _declare_qk()
        raw, stats, w, cos, sin = ctx.saved_tensors
        mod = ctx.mod
        T, blk, D = raw.shape[0], mod.blk, mod.D
        dy = torch.stack([dq.reshape(T, blk), dk.reshape(T, blk)]).contiguous()
        dw = torch.zeros(2, blk, dtype=torch.float32, device=raw.device)
        args = (raw.data_ptr(), raw.stride(0), stats.data_ptr(), stats.shape[1], w.data_ptr(), cos.data_ptr(), sin.data_ptr())
        rc = L.mm_qk_norm_rope_bwd_partials(*args, dy.data_ptr(), mod.dots_local.data_ptr(), dw.data_ptr(), T, blk, D, mod.H,
                                            mod.eps, native._st())
        native._check(rc, "qk_norm_rope_bwd_partials")
        # the row dot product runs over ALL channels: every rank's partial table goes into its slot on every rank
        nb = mod.dots_local.numel() * 4
        mod.arena.barrier()                               # the slots' previous contents have been consumed
        for p in range(mod.world):
            native._check(native.lib().mm_p2p_copy(mod.dots_peer[p] + mod.rank * nb, mod.dots_local.data_ptr(), nb, 8,
                                                   native._st()), "p2p_copy(dots)")
        mod.arena.barrier()                               # all partial tables have landed
        draw = torch.empty(T, 3 * blk, dtype=raw.dtype, device=raw.device)
        rc = L.mm_qk_norm_rope_bwd(*args, dy.data_ptr(), mod.dots_slots.data_ptr(), mod.world, draw.data_ptr(),
                                   draw.stride(0), T, blk, D, mod.H, mod.eps, native._st())
        native._check(rc, "qk_norm_rope_bwd")
        draw[:, 2 * blk:].copy_(dv.reshape(T, blk))
        lo = mod.rank * blk
        dwq = torch.zeros(mod.H, dtype=torch.float32, device=raw.device)
        dwk = torch.zeros(mod.H, dtype=torch.float32, device=raw.device)
        dwq[lo:lo + blk] = dw[0]                          # the other ranks' channels get their gradient on those ranks;
        dwk[lo:lo + blk] = dw[1]                          # the sharding engine's reduction sums the pieces
        return draw, None, dwq.to(w.dtype), dwk.to(w.dtype), None, None, None


class UlyssesQKNormRope:
    """On the head owner, after ``UlyssesQKVProjection(with_stats=True)``: RMSNorm of q and k over the whole hidden vector
    (row statistics from the projection) and interleaved RoPE, one kernel forward; the backward's row dot product is
    completed across the ranks through symmetric memory.  Returns q, k, v as [S_full, heads_local, D]."""

    def __init__(self, group, device, S_full: int, blk: int, D: int, H: int, eps: float):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.blk, self.D, self.H, self.eps = blk, D, H, eps
        dev = torch.device(device)
        nb = S_full * 2 * 4
        self.arena = SymmArena(self.world * nb + 8192, group, dev)
        off = self.arena.carve(self.world * nb)
        self.dots_slots = self.arena.view(off, self.world * S_full * 2, torch.float32).view(self.world, S_full, 2)
        self.dots_peer = [b + off for b in self.arena.peer_base]
        self.dots_local = torch.empty(S_full, 2, dtype=torch.float32, device=dev)

    def __call__(self, raw, stats, wq, wk, cos, sin):
        return _QKNormRopeFn.apply(raw, stats, wq, wk, cos.float().contiguous(), sin.float().contiguous(), self)
