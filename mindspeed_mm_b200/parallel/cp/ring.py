"""Ring attention: KV blocks travel around the context-parallel ring while every rank keeps its queries.

Forward: at step s a rank attends its queries to the KV block that originated on rank (r - s) mod P, then
merges (out, lse) with the running result (online softmax); the next block is received while the current one
is computed (isend/irecv double buffering).  Backward replays the ring with the FINAL (out, lse): each block's
dq is accumulated locally, dk/dv travel with their block and arrive home after P steps.
Causal attention uses the zig-zag layout (rank r holds chunks r and 2P-1-r of 2P chunks) so that every rank
does the same amount of work: own block -> causal; blocks from lower ranks -> all queries x first half of
the keys; blocks from higher ranks -> second half of the queries x all keys.

Reference: mindspeed_mm/fsdp/distributed/context_parallel/ring_context_parallel/ring_context_parallel.py:920-1218
(forward/backward), utils.py:98-232 (RingP2P, forward_update).  Block kernels: fp32 PyTorch math on CPU,
flash-attn's fwd/bwd entry points on the GPU library tier.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------ block kernels
def _block_fwd_ref(q, k, v, scale, causal) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,Sq,N,D], k/v [B,Sk,Nkv,D] -> out [B,Sq,N,D] (fp32), lse [B,N,Sq]."""
    rep = q.shape[2] // k.shape[2]
    qf, kf, vf = q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2)
    kf, vf = kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        sq, sk = s.shape[-2:]
        s = s.masked_fill(~torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(sk - sq), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.exp(s - lse.unsqueeze(-1)) @ vf
    return o.transpose(1, 2), lse


def _block_bwd_ref(do, q, k, v, o, lse, scale, causal):
    """Gradients of one block given the GLOBAL out / lse (so probabilities are globally normalised)."""
    rep = q.shape[2] // k.shape[2]
    qf, kf, vf = q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2)
    kr, vr = kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1)
    dof, of = do.float().transpose(1, 2), o.float().transpose(1, 2)
    s = qf @ kr.transpose(-1, -2) * scale
    if causal:
        sq, sk = s.shape[-2:]
        s = s.masked_fill(~torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(sk - sq), float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = p.transpose(-1, -2) @ dof
    dp = dof @ vr.transpose(-1, -2)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kr
    dk = ds.transpose(-1, -2) @ qf
    B, N, Sk, D = dk.shape
    dk = dk.view(B, N // rep, rep, Sk, D).sum(2)
    dv = dv.view(B, N // rep, rep, Sk, -1).sum(2)
    return dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)


def _native_ok(q, k):
    from ... import ops
    return ops.get_tier() == "native" and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and k.shape[-1] == 128


def _cu(B, S, device):
    return torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=device)


def _block_fwd(q, k, v, scale, causal):
    if q.is_cuda and _native_ok(q, k):
        from ...ops import native
        B, Sq, N, D = q.shape
        Sk = k.shape[1]
        o, lse = native.fmha_forward(q.reshape(B * Sq, N, D), k.reshape(B * Sk, -1, D), v.reshape(B * Sk, -1, D),
                                     _cu(B, Sq, q.device), _cu(B, Sk, q.device), causal, scale)
        return o.view(B, Sq, N, D).float(), lse.view(N, B, Sq).transpose(0, 1)
    if q.is_cuda:
        from flash_attn.flash_attn_interface import _flash_attn_forward
        out = _flash_attn_forward(q, k, v, 0.0, scale, causal=causal, window_size_left=-1, window_size_right=-1,
                                  softcap=0.0, alibi_slopes=None, return_softmax=False)
        return out[0].float(), out[1][..., :q.shape[1]]
    return _block_fwd_ref(q, k, v, scale, causal)


def _block_bwd(do, q, k, v, o, lse, scale, causal):
    if q.is_cuda and _native_ok(q, k):
        from ...ops import native
        B, Sq, N, D = q.shape
        Sk = k.shape[1]
        dq, dk, dv = native.fmha_backward(do.to(q.dtype).reshape(B * Sq, N, D), q.reshape(B * Sq, N, D),
                                          k.reshape(B * Sk, -1, D), v.reshape(B * Sk, -1, D),
                                          o.to(q.dtype).reshape(B * Sq, N, D),
                                          lse.transpose(0, 1).reshape(N, B * Sq).contiguous(), _cu(B, Sq, q.device),
                                          _cu(B, Sk, q.device), causal, scale)
        return dq.view(B, Sq, N, D).float(), dk.view(B, Sk, -1, D).float(), dv.view(B, Sk, -1, D).float()
    if q.is_cuda:
        from flash_attn.flash_attn_interface import _flash_attn_backward
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_backward(do.to(q.dtype).contiguous(), q, k, v, o.to(q.dtype).contiguous(), lse.contiguous(), dq, dk, dv,
                             0.0, scale, causal, -1, -1, 0.0, None, False)
        return dq.float(), dk.float(), dv.float()
    return _block_bwd_ref(do, q, k, v, o, lse, scale, causal)


def _merge(o, lse, o_b, lse_b):
    """Online-softmax merge; o [B,S,N,D] fp32, lse [B,N,S]."""
    if o is None:
        return o_b, lse_b
    new = torch.logaddexp(lse, lse_b)
    w1 = torch.exp(lse - new).transpose(1, 2).unsqueeze(-1)
    w2 = torch.exp(lse_b - new).transpose(1, 2).unsqueeze(-1)
    return o * w1 + o_b * w2, new


# ------------------------------------------------------------------------------------------ ring transport
class RingP2P:
    """Send to the next rank, receive from the previous one (batched isend/irecv), double buffered."""

    def __init__(self, group):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.next = dist.get_global_rank(group, (self.rank + 1) % self.world)
        self.prev = dist.get_global_rank(group, (self.rank - 1) % self.world)
        self._reqs = []

    def exchange(self, send: torch.Tensor, reverse: bool = False) -> torch.Tensor:
        recv = torch.empty_like(send)
        dst, src = (self.prev, self.next) if reverse else (self.next, self.prev)
        ops = [dist.P2POp(dist.isend, send.contiguous(), dst, self.group), dist.P2POp(dist.irecv, recv, src, self.group)]
        if self.rank % 2:        # odd ranks post the receive first (avoids a send-send stall on CPU backends)
            ops.reverse()
        self._reqs = dist.batch_isend_irecv(ops)
        return recv

    def wait(self):
        for r in self._reqs:
            r.wait()
        self._reqs = []


class PeerRing:
    """Ring transport over NVLink peer memory: every rank publishes its K/V block in a symmetric-memory arena; the
    block needed at the next step is pulled into a local double buffer by a copy kernel on a side stream while the
    current block is being computed, and gradient contributions are pushed straight into a per-writer slot of the
    owner's arena (summed by the owner after one barrier).  No send / recv pairs, no NCCL."""

    _cache: dict = {}

    @classmethod
    def get(cls, group, shape, dtype, device):
        key = (id(group), tuple(shape), dtype, str(device))
        inst = cls._cache.get(key)
        if inst is None:
            if len(cls._cache) > 4:
                cls._cache.clear()
            inst = cls._cache[key] = cls(group, shape, dtype, device)
        return inst

    def __init__(self, group, shape, dtype, device):
        from ...comm.symm import SymmArena
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.shape, self.dtype = tuple(shape), dtype
        n = 1
        for d in shape:
            n *= d
        self.nbytes = n * torch.empty(0, dtype=dtype).element_size()
        self.arena = SymmArena((1 + self.world) * self.nbytes + 8192, group, torch.device(device))
        self.kv_off = self.arena.carve(self.nbytes)
        self.slot_off = [self.arena.carve(self.nbytes) for _ in range(self.world)]
        self.kv = self.arena.view(self.kv_off, n, dtype).view(shape)
        self.slots = [self.arena.view(o, n, dtype).view(shape) for o in self.slot_off]
        self.local = [torch.empty(shape, dtype=dtype, device=device) for _ in range(2)]
        self.side = torch.cuda.Stream(device)

    def publish(self, kv):
        self.arena.barrier()            # nobody still reads the previous contents
        self.kv.copy_(kv)
        self.arena.barrier()

    def _copy(self, dst_ptr, src_ptr, stream):
        from ...ops import native
        native._check(native.lib().mm_p2p_copy(dst_ptr, src_ptr, self.nbytes, 64, stream.cuda_stream), "p2p_copy")

    def fetch_async(self, src_rank: int, buf: int) -> torch.Tensor:
        """Start pulling rank ``src_rank``'s published block into local buffer ``buf`` on the side stream."""
        self.side.wait_stream(torch.cuda.current_stream())
        self._copy(self.local[buf].data_ptr(), self.arena.peer_base[src_rank] + self.kv_off, self.side)
        return self.local[buf]

    def wait(self):
        torch.cuda.current_stream().wait_stream(self.side)

    def push_grad_async(self, owner: int, dkv: torch.Tensor):
        """Write this rank's gradient contribution for ``owner``'s block into slot[self.rank] of the owner's arena."""
        dkv = dkv.to(self.dtype).contiguous()
        self.side.wait_stream(torch.cuda.current_stream())
        dkv.record_stream(self.side)
        self._copy(self.arena.peer_base[owner] + self.slot_off[self.rank], dkv.data_ptr(), self.side)

    def reduce_grads(self, own: torch.Tensor, writers) -> torch.Tensor:
        self.wait()
        self.arena.barrier()            # every contribution has landed
        total = own.float()
        for w in writers:
            total = total + self.slots[w].float()
        return total


def _peer_ring_enabled(q) -> bool:
    import os
    if not q.is_cuda or os.environ.get("MM_B200_RING", "peer") != "peer":
        return False
    from ... import ops
    return ops.get_tier() == "native"


def _step_plan(causal: bool, rank: int, src: int):
    """(q slice, kv slice, causal flag) for the block from ``src``: slices are 'all', 'first', 'second' or None."""
    if not causal:
        return "all", "all", False
    if src == rank:
        return "all", "all", True
    if src < rank:
        return "all", "first", False
    return "second", "all", False


def _half(x, which, dim=1):
    if which == "all":
        return x
    h = x.shape[dim] // 2
    return x.narrow(dim, 0, h) if which == "first" else x.narrow(dim, h, h)


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, causal, scale):
        peer = _peer_ring_enabled(q)
        kv = torch.stack([k, v]).contiguous()
        ring = PeerRing.get(group, kv.shape, kv.dtype, q.device) if peer else RingP2P(group)
        P, r = ring.world, ring.rank
        B, S, N, D = q.shape
        out = torch.zeros(B, S, N, v.shape[-1], dtype=torch.float32, device=q.device)
        lse = torch.full((B, N, S), float("-inf"), dtype=torch.float32, device=q.device)
        if peer:
            ring.publish(kv)
        for s in range(P):
            if peer:
                nxt = ring.fetch_async((r - s - 1) % P, (s + 1) & 1) if s < P - 1 else None
            else:
                nxt = ring.exchange(kv) if s < P - 1 else None
            src = (r - s) % P
            qs, ks, c = _step_plan(causal, r, src)
            qb = _half(q, qs)
            ob, lb = _block_fwd(qb.contiguous(), _half(kv[0], ks).contiguous(), _half(kv[1], ks).contiguous(), scale, c)
            if qs == "all":
                o2, l2 = _merge(out if s else None, lse if s else None, ob, lb)
                out, lse = o2, l2
            else:
                h = S // 2
                o2, l2 = _merge(out[:, h:], lse[..., h:], ob, lb)
                out = torch.cat([out[:, :h], o2], 1)
                lse = torch.cat([lse[..., :h], l2], -1)
            if nxt is not None:
                ring.wait()
                kv = nxt
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.group, ctx.causal, ctx.scale = group, causal, scale
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        if _peer_ring_enabled(q):
            return _ring_backward_peer(ctx, do, q, k, v, out, lse)
        ring = RingP2P(ctx.group)
        P, r = ring.world, ring.rank
        S = q.shape[1]
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack([k, v]).contiguous()
        dkv = torch.zeros_like(kv, dtype=torch.float32)      # gradient of the block currently held
        for s in range(P):
            src = (r - s) % P
            qs, ks, c = _step_plan(ctx.causal, r, src)
            sl = slice(None) if qs == "all" else slice(S // 2, None)
            dqb, dkb, dvb = _block_bwd(do[:, sl].contiguous(), q[:, sl].contiguous(), _half(kv[0], ks).contiguous(),
                                       _half(kv[1], ks).contiguous(), out[:, sl].contiguous(), lse[..., sl].contiguous(),
                                       ctx.scale, c)
            dq[:, sl] += dqb
            if ks == "all":
                dkv[0] += dkb
                dkv[1] += dvb
            else:
                h = kv.shape[2] // 2
                dkv[0][:, :h] += dkb
                dkv[1][:, :h] += dvb
            # pass the block and its gradient on; after P hops both are back at the owner
            both = torch.cat([kv.float(), dkv]).contiguous()
            both = ring.exchange(both)
            ring.wait()
            kv, dkv = both[:2].to(k.dtype), both[2:]
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None


def _ring_backward_peer(ctx, do, q, k, v, out, lse):
    """Backward over peer memory: blocks are pulled like in the forward; each rank pushes its dK / dV contribution
    for a remote block into the owner's arena and the owner sums the P - 1 slots after one barrier."""
    kv = torch.stack([k, v]).contiguous()
    ring = PeerRing.get(ctx.group, kv.shape, kv.dtype, q.device)
    P, r = ring.world, ring.rank
    S = q.shape[1]
    dq = torch.zeros_like(q, dtype=torch.float32)
    own = torch.zeros_like(kv, dtype=torch.float32)
    ring.publish(kv)
    cur = kv
    for s in range(P):
        nxt = ring.fetch_async((r - s - 1) % P, (s + 1) & 1) if s < P - 1 else None
        src = (r - s) % P
        qs, ks, c = _step_plan(ctx.causal, r, src)
        sl = slice(None) if qs == "all" else slice(S // 2, None)
        dqb, dkb, dvb = _block_bwd(do[:, sl].contiguous(), q[:, sl].contiguous(), _half(cur[0], ks).contiguous(),
                                   _half(cur[1], ks).contiguous(), out[:, sl].contiguous(), lse[..., sl].contiguous(),
                                   ctx.scale, c)
        dq[:, sl] += dqb
        contrib = own if src == r else torch.zeros_like(kv, dtype=torch.float32)
        if ks == "all":
            contrib[0] += dkb
            contrib[1] += dvb
        else:
            h = kv.shape[2] // 2
            contrib[0][:, :h] += dkb
            contrib[1][:, :h] += dvb
        if src != r:
            ring.push_grad_async(src, contrib)
        if nxt is not None:
            ring.wait()
            cur = nxt
    total = ring.reduce_grads(own, [w for w in range(P) if w != r])
    return dq.to(q.dtype), total[0].to(k.dtype), total[1].to(v.dtype), None, None, None


def ring_attention(q, k, v, group, causal: bool = False, softmax_scale: Optional[float] = None):
    """q/k/v: [B, S_local, N, D] (zig-zag ordered when ``causal``).  Returns [B, S_local, N, D]."""
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if group is None or dist.get_world_size(group) == 1:
        from ... import ops
        return ops.attention_dense(q, k, v, causal, scale)
    return _RingAttention.apply(q, k, v, group, causal, scale)
