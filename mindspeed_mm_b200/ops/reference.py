"""Plain-PyTorch fp32 statements of every hot op.

These are the oracles the CUDA kernels are tested against and the code path
that runs on CPU (gloo plumbing tests).  Each function upcasts to fp32, does
the arithmetic the obvious way and casts back, so that it is easy to audit.

Parity notes (reference paths are relative to the MindSpeed-MM tree):
  * rms_norm            <- torch_npu.npu_rms_norm, mindspeed_mm/fsdp/ops/npu_patch/npu_fused_operator.py:33-37
  * swiglu              <- mindspeed_mm/fsdp/ops/swiglu.py:8-31
  * rope_rotate_half    <- mindspeed_mm/models/vision/vision_encoders/qwen2vl_vit_model.py:48-67
  * rope_interleaved    <- mindspeed_mm/models/predictor/dits/wan_dit.py:871-885
  * layer_norm_modulate <- mindspeed_mm/models/predictor/dits/wan_dit.py:764-766
  * attention_varlen    <- torch_npu.npu_fusion_attention TND layout, mindspeed_mm/fsdp/ops/flash_attn/flash_attn.py:511-526
  * linear_cross_entropy<- mindspeed_mm/fsdp/features/memory/chunkloss/chunkloss.py:98-154
  * grouped_gemm        <- mindspeed_mm/fsdp/ops/moe_ops/gemm.py:35-92
  * permute/unpermute   <- mindspeed_mm/fsdp/ops/moe_ops/permute.py:8-16, unpermute.py:8-21
  * gated delta rule    <- mindspeed_mm/fsdp/models/qwen3_5_moe/modeling_qwen3_5_moe.py:408-527
  * causal_conv1d       <- mindspeed_mm/fsdp/ops/gdn/triton/convolution.py:42
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def layer_norm(x, weight=None, bias=None, eps: float = 1e-6):
    y = F.layer_norm(x.float(), (x.shape[-1],), None if weight is None else weight.float(),
                     None if bias is None else bias.float(), eps)
    return y.to(x.dtype)


def layer_norm_modulate(x, scale, shift, eps: float = 1e-6):
    """adaLN: LayerNorm without affine, then ``y * (1 + scale) + shift`` (scale/shift broadcast over S)."""
    y = F.layer_norm(x.float(), (x.shape[-1],), None, None, eps)
    return (y * (1.0 + scale.float()) + shift.float()).to(x.dtype)


def gated_residual(x, y, gate):
    """``x + gate * y`` with fp32 accumulation (adaLN-zero residual)."""
    return (x.float() + gate.float() * y.float()).to(x.dtype)


def l2_norm(x, eps: float = 1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def gated_rms_norm(x, z, weight, eps: float = 1e-6):
    """``rmsnorm(x) * weight * silu(z)`` (GDN output norm)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return (y * F.silu(z.float())).to(x.dtype)


# --------------------------------------------------------------------------- activations
def swiglu(gate_up: torch.Tensor, clamp: Optional[float] = None) -> torch.Tensor:
    """``silu(a) * b`` where ``gate_up = [a | b]`` along the last dim."""
    a, b = gate_up.float().chunk(2, dim=-1)
    if clamp is not None:
        a = a.clamp(max=clamp)
        b = b.clamp(min=-clamp, max=clamp)
    return (F.silu(a) * b).to(gate_up.dtype)


def gelu_tanh(x):
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


# --------------------------------------------------------------------------- rotary embeddings
def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope_rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-rotation RoPE.  x: [T, N, D]; cos/sin: [T, D] (already duplicated over both halves)."""
    xf = x.float()
    c = cos.float().unsqueeze(-2)
    s = sin.float().unsqueeze(-2)
    return (xf * c + _rotate_half(xf) * s).to(x.dtype)


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair (complex) RoPE used by Wan.  x: [T, N, D]; cos/sin: [T, D/2]."""
    xf = x.float()
    xr, xi = xf[..., 0::2], xf[..., 1::2]
    c = cos.float().unsqueeze(-2)
    s = sin.float().unsqueeze(-2)
    out = torch.stack((xr * c - xi * s, xr * s + xi * c), dim=-1).flatten(-2)
    return out.to(x.dtype)


def mrope_cos_sin(position_ids: torch.Tensor, head_dim: int, theta: float,
                  mrope_section: Sequence[int], dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Multimodal RoPE tables.  position_ids: [3, T] (t, h, w).  Returns cos, sin: [T, head_dim].

    Frequency band i of the half-dim takes its position from axis ``axis(i)`` where the
    first ``mrope_section[0]`` bands follow t, the next ``[1]`` follow h, the rest follow w.
    """
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=position_ids.device) / half))
    freqs = position_ids.float().unsqueeze(-1) * inv_freq  # [3, T, half]
    sel = torch.zeros(half, dtype=torch.long, device=position_ids.device)
    start = 0
    for axis, n in enumerate(mrope_section):
        sel[start:start + n] = axis
        start += n
    f = torch.gather(freqs, 0, sel.view(1, 1, half).expand(1, freqs.shape[1], half)).squeeze(0)  # [T, half]
    emb = torch.cat((f, f), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rope3d_freqs(grid: Tuple[int, int, int], head_dim: int, theta: float = 10000.0, device=None):
    """Wan 3-D RoPE tables for a (F, H, W) token grid.  Returns cos, sin: [F*H*W, head_dim/2].

    The head dim is split into (d - 4*(d//6), 2*(d//6), 2*(d//6)) channels for (f, h, w) (44/42/42 for
    d = 128); each part is rotated as interleaved pairs at its own axis position.
    """
    f, h, w = grid
    d = head_dim
    dims = (d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6))
    outs = []
    for n, dim in zip((f, h, w), dims):
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device)[: dim // 2] / dim))
        outs.append(torch.outer(torch.arange(n, dtype=torch.float64, device=device), inv))
    ff = outs[0].view(f, 1, 1, -1).expand(f, h, w, -1)
    hh = outs[1].view(1, h, 1, -1).expand(f, h, w, -1)
    ww = outs[2].view(1, 1, w, -1).expand(f, h, w, -1)
    ang = torch.cat((ff, hh, ww), dim=-1).reshape(f * h * w, -1)
    return ang.cos().float(), ang.sin().float()


# --------------------------------------------------------------------------- attention
def attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal: bool = False,
                     softmax_scale: Optional[float] = None, return_lse: bool = False):
    """Packed (TND) attention with GQA.  q: [Tq, Nq, D], k/v: [Tk, Nkv, D]; int cu_seqlens.

    Segments are independent; ``causal`` aligns the bottom-right corner like flash-attn.
    """
    Tq, Nq, D = q.shape
    Nkv = k.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty(Tq, Nq, v.shape[-1], dtype=torch.float32, device=q.device)
    lse = torch.empty(Nq, Tq, dtype=torch.float32, device=q.device)
    cq = [int(c) for c in cu_seqlens_q]
    ck = [int(c) for c in cu_seqlens_k]
    rep = Nq // Nkv
    for i in range(len(cq) - 1):
        qs = q[cq[i]:cq[i + 1]].float().transpose(0, 1)  # [Nq, sq, D]
        ks = k[ck[i]:ck[i + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[ck[i]:ck[i + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.matmul(qs, ks.transpose(1, 2)) * scale
        if causal:
            sq, sk = s.shape[-2:]
            mask = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(diagonal=sk - sq)
            s = s.masked_fill(~mask, float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l.unsqueeze(-1))
        out[cq[i]:cq[i + 1]] = torch.matmul(p, vs).transpose(0, 1)
        lse[:, cq[i]:cq[i + 1]] = l
    out = out.to(q.dtype)
    return (out, lse) if return_lse else out


def attention_dense(q, k, v, causal=False, softmax_scale=None, return_lse=False):
    """Batched BSND attention (DiT path).  q: [B, Sq, N, D], k/v: [B, Sk, Nkv, D]."""
    B, Sq, N, D = q.shape
    Sk = k.shape[1]
    cq = torch.arange(0, (B + 1) * Sq, Sq)
    ck = torch.arange(0, (B + 1) * Sk, Sk)
    r = attention_varlen(q.reshape(B * Sq, N, D), k.reshape(B * Sk, -1, D), v.reshape(B * Sk, -1, v.shape[-1]),
                         cq, ck, causal, softmax_scale, return_lse)
    if return_lse:
        return r[0].view(B, Sq, N, -1), r[1].view(N, B, Sq).transpose(0, 1)
    return r.view(B, Sq, N, -1)


def merge_attention_states(o1, lse1, o2, lse2):
    """Online-softmax merge of two partial attention results (ring attention step).

    o*: [T, N, D], lse*: [N, T].  Mirrors ``forward_update`` in
    fsdp/distributed/context_parallel/ring_context_parallel/utils.py:185.
    """
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).transpose(0, 1).unsqueeze(-1)
    w2 = torch.exp(lse2 - lse).transpose(0, 1).unsqueeze(-1)
    return (o1.float() * w1 + o2.float() * w2).to(o1.dtype), lse


# --------------------------------------------------------------------------- loss
def linear_cross_entropy(h, weight, labels, ignore_index: int = -100, reduction: str = "sum"):
    """``CE(h @ weight.T, labels)`` in fp32; returns (loss, n_valid)."""
    logits = h.float() @ weight.float().t()
    loss = F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction=reduction)
    return loss, (labels != ignore_index).sum()


# --------------------------------------------------------------------------- MoE
def grouped_gemm(x, w, counts):
    """x: [sum(counts), K]; w: [E, K, N]; rows of x are grouped by expert in order."""
    outs, s = [], 0
    for e, c in enumerate([int(c) for c in counts]):
        outs.append(x[s:s + c].float() @ w[e].float())
        s += c
    return torch.cat(outs, 0).to(x.dtype) if outs else x.new_zeros(0, w.shape[-1])


def moe_permute(tokens, topk_ids, num_experts: Optional[int] = None):
    """Stable sort of the T*k (token, slot) pairs by expert id.

    Returns (permuted [T*k, H], sorted_indices [T*k] into the flattened (token, slot) axis).
    """
    T, k = topk_ids.shape
    flat = topk_ids.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    return tokens.index_select(0, order // k), order


def moe_unpermute(permuted, order, probs):
    """Inverse of :func:`moe_permute` with prob-weighted sum over the k slots."""
    T, k = probs.shape
    out = torch.zeros(T * k, permuted.shape[-1], dtype=torch.float32, device=permuted.device)
    out.index_copy_(0, order, permuted.float())
    return (out.view(T, k, -1) * probs.float().unsqueeze(-1)).sum(1).to(permuted.dtype)


# --------------------------------------------------------------------------- GDN
def causal_conv1d(x, weight, bias=None, activation: Optional[str] = "silu", cu_seqlens=None):
    """Depthwise causal conv.  x: [T, D] packed (or [B, T, D]); weight: [D, K]."""
    squeeze = x.dim() == 2
    if squeeze:
        x = x.unsqueeze(0)
    B, T, D = x.shape
    K = weight.shape[-1]
    xf = x.float()
    out = torch.zeros_like(xf)
    bounds = [0, T] if cu_seqlens is None else [int(c) for c in cu_seqlens]
    for i in range(len(bounds) - 1):
        seg = xf[:, bounds[i]:bounds[i + 1]].transpose(1, 2)  # [B, D, t]
        y = F.conv1d(F.pad(seg, (K - 1, 0)), weight.float().unsqueeze(1), None if bias is None else bias.float(), groups=D)
        out[:, bounds[i]:bounds[i + 1]] = y.transpose(1, 2)
    if activation == "silu":
        out = F.silu(out)
    out = out.to(x.dtype)
    return out.squeeze(0) if squeeze else out


def gated_delta_rule_recurrent(q, k, v, g, beta, scale=None, initial_state=None):
    """Token-by-token gated delta rule.  q,k: [B,T,H,K]; v: [B,T,H,V]; g,beta: [B,T,H].

    S_t = S_{t-1} * exp(g_t);  S_t += k_t (beta_t (v_t - S_t^T k_t))^T;  o_t = S_t^T q_t * scale
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    S = torch.zeros(B, H, K, V, device=q.device) if initial_state is None else initial_state.float().clone()
    o = torch.empty(B, T, H, V, device=q.device)
    for t in range(T):
        S = S * g[:, t].exp()[..., None, None]
        kv = torch.einsum("bhk,bhkv->bhv", k[:, t], S)
        delta = (v[:, t] - kv) * beta[:, t][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], delta)
        o[:, t] = torch.einsum("bhk,bhkv->bhv", q[:, t] * scale, S)
    return o, S


def gated_delta_rule_chunked(q, k, v, g, beta, scale=None, chunk: int = 64, initial_state=None):
    """Chunk-parallel gated delta rule (WY form); same math as the recurrent form.

    Stages: g cumsum -> A = -(beta K K^T * decay) strictly lower -> (I - A)^-1 by forward
    substitution -> u = T (v beta), w = T (k beta e^g) -> per-chunk state update -> output.
    """
    B, T0, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    pad = (-T0) % chunk
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
    T = T0 + pad
    n = T // chunk
    # [B,H,n,C,*]
    rs = lambda t: t.transpose(1, 2).reshape(B, H, n, chunk, -1)
    q, k, v = rs(q) * scale, rs(k), rs(v)
    g = g.transpose(1, 2).reshape(B, H, n, chunk)
    beta = beta.transpose(1, 2).reshape(B, H, n, chunk)
    gc = g.cumsum(-1)
    decay = (gc.unsqueeze(-1) - gc.unsqueeze(-2)).tril().exp().tril()
    kb = k * beta.unsqueeze(-1)
    vb = v * beta.unsqueeze(-1)
    A = -(kb @ k.transpose(-1, -2) * decay).tril(-1)
    # (I - A)^-1 via row-wise forward substitution
    rows = [A[..., 0, :]]                         # built out of place so that autograd can differentiate it
    for i in range(1, chunk):
        a = A[..., i, :i]
        prev = torch.stack(rows, dim=-2)[..., :i]
        rows.append(F.pad(a + (a.unsqueeze(-1) * prev).sum(-2), (0, chunk - i)))
    Tm = torch.stack(rows, dim=-2) + torch.eye(chunk, device=q.device)
    u = Tm @ vb
    w = Tm @ (kb * gc.exp().unsqueeze(-1))
    S = torch.zeros(B, H, K, V, device=q.device) if initial_state is None else initial_state.float().clone()
    o = torch.empty(B, H, n, chunk, V, device=q.device)
    for c in range(n):
        v_new = u[:, :, c] - w[:, :, c] @ S
        inter = (q[:, :, c] * gc[:, :, c].exp().unsqueeze(-1)) @ S
        attn = (q[:, :, c] @ k[:, :, c].transpose(-1, -2) * decay[:, :, c]).tril()
        o[:, :, c] = inter + attn @ v_new
        last = gc[:, :, c, -1]
        S = S * last.exp()[..., None, None] + (k[:, :, c] * (last.unsqueeze(-1) - gc[:, :, c]).exp().unsqueeze(-1)).transpose(-1, -2) @ v_new
    o = o.reshape(B, H, T, V).transpose(1, 2)[:, :T0]
    return o, S


def kda_recurrent(q, k, v, g, beta, scale=None, initial_state=None):
    """Kimi delta attention, token by token: the delta rule with a per-channel gate.

    q, k, g: [B,T,H,K] (g = log decay per key channel); v: [B,T,H,V]; beta: [B,T,H].
    S_t = diag(exp(g_t)) S_{t-1};  S_t += k_t (beta_t (v_t - S_t^T k_t))^T;  o_t = S_t^T q_t * scale
    (naive form of the reference: mindspeed_mm/fsdp/ops/kda/chunk_kda_naive.py).
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    S = torch.zeros(B, H, K, V, device=q.device) if initial_state is None else initial_state.float().clone()
    outs = []
    for t in range(T):
        S = S * g[:, t].exp().unsqueeze(-1)
        kv = torch.einsum("bhk,bhkv->bhv", k[:, t], S)
        delta = (v[:, t] - kv) * beta[:, t][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], delta)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t] * scale, S))
    return torch.stack(outs, 1), S


def kda_chunked(q, k, v, g, beta, scale=None, chunk: int = 64, initial_state=None):
    """Chunk-parallel KDA (WY form with per-channel decay); same math as :func:`kda_recurrent`.

    Inside a chunk the pairwise decay exp(G_i - G_j) is applied per key channel by folding exp(G) into one operand
    and exp(-G) into the other; ``g`` is accumulated from the chunk start, so the exponents stay bounded by the
    chunk's total decay.
    """
    B, T0, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    pad = (-T0) % chunk
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    if pad:
        q, k, v, g = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v, g))
        beta = F.pad(beta, (0, 0, 0, pad))
    n = (T0 + pad) // chunk
    rs = lambda t: t.transpose(1, 2).reshape(B, H, n, chunk, -1)
    q, k, v, g = rs(q) * scale, rs(k), rs(v), rs(g)
    beta = beta.transpose(1, 2).reshape(B, H, n, chunk)
    G = g.cumsum(-2)                                          # [B,H,n,C,K]
    k_up, k_dn, q_up = k * G.exp(), k * (-G).exp(), q * G.exp()
    eye = torch.eye(chunk, device=q.device)
    A = ((k_up * beta.unsqueeze(-1)) @ k_dn.transpose(-1, -2)).tril(-1)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False, unitriangular=True)
    u = Tm @ (v * beta.unsqueeze(-1))
    w = Tm @ (k_up * beta.unsqueeze(-1))
    attn = (q_up @ k_dn.transpose(-1, -2)).tril()
    last = G[..., -1:, :]                                     # [B,H,n,1,K]
    k_tail = k * (last - G).exp()
    S = torch.zeros(B, H, K, V, device=q.device) if initial_state is None else initial_state.float().clone()
    outs = []
    for c in range(n):
        v_new = u[:, :, c] - w[:, :, c] @ S
        outs.append(q_up[:, :, c] @ S + attn[:, :, c] @ v_new)
        S = S * last[:, :, c].transpose(-1, -2).exp() + k_tail[:, :, c].transpose(-1, -2) @ v_new
    o = torch.stack(outs, 2).reshape(B, H, n * chunk, V).transpose(1, 2)[:, :T0]
    return o, S


# --------------------------------------------------------------------------- optimizer
def adamw_step(p32, m, v, grad, lr, beta1, beta2, eps, wd, step, grad_scale: float = 1.0, p16=None):
    """One decoupled-weight-decay Adam update on fp32 master weights (in place)."""
    g = grad.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    p32.mul_(1 - lr * wd)
    denom = (v / bc2).sqrt_().add_(eps)
    p32.addcdiv_(m / bc1, denom, value=-lr)
    if p16 is not None:
        p16.copy_(p32)
