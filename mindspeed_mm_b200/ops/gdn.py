"""Chunked gated delta rule on packed sequences: batched prologue + sequential state pass.

The WY form splits the operator in two:

* ``chunk_prologue`` -- everything local to a 64-token chunk (cumulative gates, the unit-triangular solve, ``u``,
  ``w``, the decayed ``q`` / ``k`` and the masked intra-chunk attention).  It is plain batched PyTorch over all
  chunks of all sequences at once, so autograd differentiates it.
* ``state_pass`` -- the walk over the chunks of a sequence, each needing the state its predecessor left.  On a GPU
  the forward is the tcgen05 kernel of ``csrc/gdn.cu`` (state resident in tensor memory); on CPU a PyTorch loop with
  the same inputs and outputs.  Its backward is written by hand: only ``dS`` has to be walked backwards over the
  chunks, every other gradient is a batched product of saved per-chunk states.

Operator parity: fla ``chunk_gated_delta_rule`` as called by the reference's Qwen3.5 gated-delta-net block
(fsdp/models/qwen3_5/modeling_qwen3_5.py) with ``cu_seqlens`` packing.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

CHUNK = 64


# ------------------------------------------------------------------------------------------ chunk layout
class ChunkLayout:
    """Maps packed tokens [T] to chunk-padded slots [NC * 64]; chunks never straddle a sequence."""

    def __init__(self, cu_seqlens: Sequence[int], device):
        cu = [int(c) for c in cu_seqlens]
        self.T = cu[-1]
        slot_of_tok: List[torch.Tensor] = []
        seq_chunks = [0]
        pos: List[int] = []
        seq_of: List[int] = []
        for s, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
            n = (b - a + CHUNK - 1) // CHUNK
            slot_of_tok.append(torch.arange(b - a) + seq_chunks[-1] * CHUNK)
            pos += list(range(n))
            seq_of += [s] * n
            seq_chunks.append(seq_chunks[-1] + n)
        self.NC = seq_chunks[-1]
        self.nseq = len(cu) - 1
        # first packed token and number of valid tokens of every chunk (for the prologue kernel, which reads the packed
        # tensors directly)
        tok0 = [a + j * CHUNK for a, b in zip(cu[:-1], cu[1:]) for j in range((b - a + CHUNK - 1) // CHUNK)]
        clen = [min(CHUNK, b - a - j * CHUNK) for a, b in zip(cu[:-1], cu[1:]) for j in range((b - a + CHUNK - 1) // CHUNK)]
        self.chunk_tok0 = torch.tensor(tok0, dtype=torch.int32, device=device)
        self.chunk_len = torch.tensor(clen, dtype=torch.int32, device=device)
        self.max_chunks = max(pos) + 1 if pos else 0
        self.slot_of_tok = torch.cat(slot_of_tok).to(device) if slot_of_tok else torch.zeros(0, dtype=torch.long, device=device)
        self.seq_chunks = torch.tensor(seq_chunks, dtype=torch.int32, device=device)
        self.seq_chunks_host = seq_chunks
        # chunks at position j of their sequence (and the sequences they belong to), for the backward walk
        self.idx_at = [torch.tensor([c for c, pj in enumerate(pos) if pj == j], dtype=torch.long, device=device)
                       for j in range(self.max_chunks)]
        self.seq_at = [torch.tensor([seq_of[c] for c, pj in enumerate(pos) if pj == j], dtype=torch.long, device=device)
                       for j in range(self.max_chunks)]

    def scatter(self, x: torch.Tensor) -> torch.Tensor:
        """[T, H, ...] -> [H, NC, 64, ...] with zero padding."""
        out = x.new_zeros((self.NC * CHUNK,) + tuple(x.shape[1:]))
        out = out.index_copy(0, self.slot_of_tok, x)
        out = out.view((self.NC, CHUNK) + tuple(x.shape[1:]))
        return out.movedim(2, 0)

    def gather(self, y: torch.Tensor) -> torch.Tensor:
        """[H, NC*64, V] -> [T, H, V]."""
        return y.transpose(0, 1).index_select(0, self.slot_of_tok)


# ------------------------------------------------------------------------------------------ prologue
def chunk_prologue(q, k, v, g, beta, scale: float):
    """Inputs [H, NC, 64, *] (fp32).  Returns W, Qg, Kd [H,NC,64,K], At [H,NC,64,64], U [H,NC,64,V], gamma [H,NC]."""
    gc = g.cumsum(-1)
    diff = gc.unsqueeze(-1) - gc.unsqueeze(-2)
    tril = torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=q.device).tril()
    decay = torch.where(tril, diff, torch.full_like(diff, -float("inf"))).exp()
    kb = k * beta.unsqueeze(-1)
    A = (kb @ k.transpose(-1, -2) * decay).tril(-1)              # I + A is the unit-triangular system
    eye = torch.eye(CHUNK, device=q.device, dtype=q.dtype)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False, unitriangular=True)
    U = Tm @ (v * beta.unsqueeze(-1))
    W = Tm @ (kb * gc.exp().unsqueeze(-1))
    Qg = q * (scale * gc.exp()).unsqueeze(-1)
    last = gc[..., -1:]
    Kd = k * (last - gc).exp().unsqueeze(-1)
    At = (q @ k.transpose(-1, -2)) * (decay * scale)
    gamma = last.squeeze(-1).exp()
    return W, Qg, Kd, At, U, gamma


# ------------------------------------------------------------------------------------------ state pass
def _state_pass_torch(W, Qg, Kd, At, U, gamma, layout: ChunkLayout):
    """PyTorch state walk with the kernel's contract.  Shapes [H, NC, 64, *]; returns O, Vn, SprevT."""
    H, NC, _, K = W.shape
    V = U.shape[-1]
    O = torch.empty(H, NC, CHUNK, V, dtype=torch.float32, device=W.device)
    Vn = torch.empty_like(O)
    SprevT = torch.empty(H, NC, V, K, dtype=torch.float32, device=W.device)
    sc = layout.seq_chunks_host
    Wf, Qf, Kf, Af, Uf = (t.float() for t in (W, Qg, Kd, At, U))
    for s in range(layout.nseq):
        S = torch.zeros(H, K, V, dtype=torch.float32, device=W.device)
        for c in range(sc[s], sc[s + 1]):
            SprevT[:, c] = S.transpose(-1, -2)
            vn = Uf[:, c] - Wf[:, c] @ S
            O[:, c] = Qf[:, c] @ S + Af[:, c] @ vn
            Vn[:, c] = vn
            S = S * _decay(gamma[:, c]) + Kf[:, c].transpose(-1, -2) @ vn
    return O, Vn, SprevT


def _decay(g: torch.Tensor) -> torch.Tensor:
    """Decay of one chunk, broadcast over the [H, K, V] state: [H] (one factor per head) or [H, K] (one per key channel)."""
    return g[:, None, None] if g.dim() == 1 else g[:, :, None]


def _state_pass_native(W, Qg, Kd, At, U, gamma, layout: ChunkLayout, want_saved: bool):
    from . import native
    H, NC, _, K = W.shape
    V = U.shape[-1]
    dev = W.device
    O = torch.empty(H, NC, CHUNK, V, dtype=torch.bfloat16, device=dev)
    Vn = torch.empty_like(O) if want_saved else None
    SprevT = torch.empty(H, NC, V, K, dtype=torch.bfloat16, device=dev) if want_saved else None
    native._check(native.lib().mm_gdn_fwd(
        W.data_ptr(), Qg.data_ptr(), Kd.data_ptr(), At.data_ptr(), U.data_ptr(), gamma.data_ptr(),
        layout.seq_chunks.data_ptr(), O.data_ptr(), Vn.data_ptr() if want_saved else None,
        SprevT.data_ptr() if want_saved else None, None, H, NC, layout.nseq, int(gamma.dim() == 3),
        native.status_word(dev).data_ptr(), native._st()), "gdn_fwd")
    return O, Vn, SprevT


class _StatePass(torch.autograd.Function):
    @staticmethod
    def forward(ctx, W, Qg, Kd, At, U, gamma, layout):
        need = any(t.requires_grad for t in (W, Qg, Kd, At, U, gamma))
        if W.is_cuda:
            args = [t.to(torch.bfloat16).contiguous() for t in (W, Qg, Kd, At, U)]
            gam = gamma.float().contiguous()
            O, Vn, SprevT = _state_pass_native(*args, gam, layout, need)
            saved = args + [gam]
        else:
            O, Vn, SprevT = _state_pass_torch(W, Qg, Kd, At, U, gamma, layout)
            saved = [W, Qg, Kd, At, U, gamma]
        if need:
            ctx.save_for_backward(*saved[:4], saved[5], Vn, SprevT)
        ctx.layout = layout
        ctx.in_dtypes = [t.dtype for t in (W, Qg, Kd, At, U, gamma)]
        return O

    @staticmethod
    def backward(ctx, dO):
        W, Qg, Kd, At, gamma, Vn, SprevT = ctx.saved_tensors
        lay: ChunkLayout = ctx.layout
        H, NC, _, K = W.shape
        V = Vn.shape[-1]
        dev = W.device
        cdt = W.dtype                       # bf16 on a GPU (tensor-core batched products), fp32 on CPU
        dO = dO.to(cdt)
        if W.is_cuda and _native_bwd_ok():
            # the walk over the chunks (last to first) is one kernel per (sequence, head): tcgen05, gradient state in TMEM
            from . import native
            dOb = dO.to(torch.bfloat16).contiguous()
            dVn = torch.empty(H, NC, CHUNK, V, dtype=torch.bfloat16, device=dev)
            GnT = torch.empty(H, NC, V, K, dtype=torch.bfloat16, device=dev)
            native._check(native.lib().mm_gdn_bwd(
                W.data_ptr(), Qg.data_ptr(), Kd.data_ptr(), At.data_ptr(), dOb.data_ptr(), gamma.data_ptr(),
                lay.seq_chunks.data_ptr(), dVn.data_ptr(), GnT.data_ptr(), H, NC, lay.nseq, int(gamma.dim() == 3),
                native.status_word(dev).data_ptr(), native._st()), "gdn_bwd")
            dSn_all = GnT.transpose(-1, -2)
        else:
            dVn = torch.empty(H, NC, CHUNK, V, dtype=cdt, device=dev)
            dSn_all = torch.empty(H, NC, K, V, dtype=cdt, device=dev)     # gradient w.r.t. the state after each chunk
            dS_seq = torch.zeros(H, lay.nseq, K, V, dtype=torch.float32, device=dev)
            QgT_dO = Qg.transpose(-1, -2) @ dO                            # [H, NC, K, V]   batched once
            AtT_dO = At.transpose(-1, -2) @ dO                            # [H, NC, 64, V]
            for j in range(lay.max_chunks - 1, -1, -1):
                idx, sidx = lay.idx_at[j], lay.seq_at[j]
                dSn = dS_seq[:, sidx]                                     # fp32 [H, n, K, V]
                dSn_c = dSn.to(cdt)
                dSn_all[:, idx] = dSn_c
                dvn = AtT_dO[:, idx] + Kd[:, idx] @ dSn_c
                dVn[:, idx] = dvn
                gam = gamma[:, idx, None, None] if gamma.dim() == 2 else gamma[:, idx, :, None]
                dS_prev = QgT_dO[:, idx].float() + gam * dSn - (W[:, idx].transpose(-1, -2) @ dvn).float()
                dS_seq[:, sidx] = dS_prev
        dU = dVn
        dW = -(dVn @ SprevT.to(cdt))                                  # [64, V] @ [V, K]
        dQg = dO @ SprevT.to(cdt)
        dAt = dO @ Vn.to(cdt).transpose(-1, -2)
        dKd = Vn.to(cdt) @ dSn_all.transpose(-1, -2)
        dgamma = (dSn_all.float() * SprevT.float().transpose(-1, -2)).sum((-1, -2) if gamma.dim() == 2 else -1)
        outs = (dW, dQg, dKd, dAt, dU, dgamma)
        return tuple(o.to(dt) for o, dt in zip(outs, ctx.in_dtypes)) + (None,)


def _native_bwd_ok() -> bool:
    """The backward walk kernel: on unless ``MM_B200_GDN_BWD_KERNEL=0`` (the PyTorch loop then runs instead)."""
    import os
    from . import native
    native.lib()
    return os.environ.get("MM_B200_GDN_BWD_KERNEL", "1") != "0" and native._STATUS.get("mm_gdn_bwd", False)


def state_pass(W, Qg, Kd, At, U, gamma, layout: ChunkLayout):
    return _StatePass.apply(W, Qg, Kd, At, U, gamma, layout)


# ------------------------------------------------------------------------------------------ public
_layout_cache: dict = {}


def _layout(cu_seqlens, device) -> ChunkLayout:
    cu = cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens
    key = (tuple(int(c) for c in cu), str(device))
    lay = _layout_cache.get(key)
    if lay is None:
        if len(_layout_cache) > 64:
            _layout_cache.clear()
        lay = _layout_cache[key] = ChunkLayout(key[0], device)
    return lay


def gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, scale: Optional[float] = None):
    """q, k: [T, H, K]; v: [T, H, V]; g (log gate), beta: [T, H].  Returns [T, H, V] in ``v.dtype``."""
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    lay = _layout(cu_seqlens, q.device)
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, g, beta))
    if q.is_cuda and not needs_grad and K == 128 and v.shape[-1] == 128 and _native_tier():
        # a pass that keeps no graph (inference, the first forward of a recomputed layer): the chunk-local prologue is one
        # kernel that reads the packed tensors, then the tcgen05 state pass; nothing is scattered to a padded layout first
        return _forward_native(q, k, v, g, beta, lay, scale)
    qc, kc, vc = (lay.scatter(t.float()) for t in (q, k, v))
    gcn, bc = (lay.scatter(t.float()) for t in (g, beta))
    W, Qg, Kd, At, U, gamma = chunk_prologue(qc, kc, vc, gcn, bc, scale)
    O = state_pass(W, Qg, Kd, At, U, gamma, lay)
    H, NC = O.shape[:2]
    return lay.gather(O.reshape(H, NC * CHUNK, -1)).to(v.dtype)


def _native_tier() -> bool:
    from . import get_tier
    return get_tier() == "native"


def _forward_native(q, k, v, g, beta, lay: ChunkLayout, scale: float):
    from . import native
    T, H, K = q.shape
    V = v.shape[-1]
    dev, NC = q.device, lay.NC
    qb, kb, vb = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
    gf, bf = g.float().contiguous(), beta.float().contiguous()
    W, Qg, Kd, U = (torch.empty(H, NC, CHUNK, K if i < 3 else V, dtype=torch.bfloat16, device=dev) for i in range(4))
    At = torch.empty(H, NC, CHUNK, CHUNK, dtype=torch.bfloat16, device=dev)
    gamma = torch.empty(H, NC, dtype=torch.float32, device=dev)
    native._check(native.lib().mm_gdn_prologue(
        qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), gf.data_ptr(), bf.data_ptr(), lay.chunk_tok0.data_ptr(),
        lay.chunk_len.data_ptr(), W.data_ptr(), Qg.data_ptr(), Kd.data_ptr(), At.data_ptr(), U.data_ptr(), gamma.data_ptr(),
        H, NC, float(scale), native._st()), "gdn_prologue")
    O, _, _ = _state_pass_native(W, Qg, Kd, At, U, gamma, lay, False)
    return lay.gather(O.reshape(H, NC * CHUNK, -1)).to(v.dtype)


def kda_chunk_prologue(q, k, v, g, beta, scale: float):
    """Kimi delta attention: ``g`` [H, NC, 64, K] is a log decay per key channel.  Same outputs as ``chunk_prologue``
    with gamma [H, NC, K].  The pairwise decay exp(G_i - G_j) is applied per channel by folding exp(G) into one operand
    and exp(-G) into the other (G accumulated from the chunk start, so the exponents are bounded by the chunk's decay)."""
    G = g.cumsum(-2)
    up, dn = G.exp(), (-G).exp()
    k_up, k_dn = k * up, k * dn
    kb_up = k_up * beta.unsqueeze(-1)
    A = (kb_up @ k_dn.transpose(-1, -2)).tril(-1)
    eye = torch.eye(CHUNK, device=q.device, dtype=q.dtype)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False, unitriangular=True)
    U = Tm @ (v * beta.unsqueeze(-1))
    W = Tm @ kb_up
    Qg = q * up * scale
    last = G[..., -1:, :]
    Kd = k * (last - G).exp()
    At = (Qg @ k_dn.transpose(-1, -2)).tril()
    return W, Qg, Kd, At, U, last.squeeze(-2).exp()


def kimi_delta_attention_varlen(q, k, v, g, beta, cu_seqlens, scale: Optional[float] = None):
    """q, k, g: [T, H, K] (g = log decay per key channel); v: [T, H, V]; beta: [T, H].  Returns [T, H, V] in ``v.dtype``.
    Same operator as the reference's chunked KDA (fsdp/ops/kda/chunk_kda_naive.py) on packed sequences: batched
    chunk-local prologue, then the state walk of the gated delta rule with one decay per key channel."""
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    lay = _layout(cu_seqlens, q.device)
    qc, kc, vc, gc_ = (lay.scatter(t.float()) for t in (q, k, v, g))
    bc = lay.scatter(beta.float())
    W, Qg, Kd, At, U, gamma = kda_chunk_prologue(qc, kc, vc, gc_, bc, scale)
    O = state_pass(W, Qg, Kd, At, U, gamma, lay)
    H, NC = O.shape[:2]
    return lay.gather(O.reshape(H, NC * CHUNK, -1)).to(v.dtype)


def supported(q, v, chunk: int) -> bool:
    return chunk == CHUNK and q.shape[-1] == 128 and v.shape[-1] == 128
