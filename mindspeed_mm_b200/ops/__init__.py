"""Hot-op front end.

Every model in the package calls the functions below, never ``torch.nn.functional``
directly, so that one switch decides what executes:

* CPU tensors           -> :mod:`.reference` (plain fp32 PyTorch; what the gloo tests run)
* CUDA tensors, ``native``  tier -> hand-written sm_100a kernels from ``csrc/`` (:mod:`.native`)
* CUDA tensors, ``library`` tier -> cuBLAS / flash-attn / torch eager.  This is the
  "NCCL + cuBLAS" baseline tier the native kernels are measured against.

The tier is process-global (``set_tier``) and defaults to ``native`` on a GPU.  On a GPU
box the native tier refuses to run if the compiled extension is missing, so a silent
fallback cannot pass for the product.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import reference as ref

_TIER = os.environ.get("MM_B200_TIER", "native")
_STRICT = os.environ.get("MM_B200_STRICT", "0") == "1"
# op name -> number of calls that were handed CUDA tensors on the native tier and did NOT run a kernel of this
# package (library or eager PyTorch instead).  Benchmarks print it; ``set_strict(True)`` turns a count into an error.
FALLBACKS: dict = {}


def set_tier(tier: str) -> None:
    global _TIER
    if tier not in ("native", "library"):
        raise ValueError(f"unknown op tier {tier!r}")
    _TIER = tier


def get_tier() -> str:
    return _TIER


def set_strict(on: bool = True) -> None:
    """Strict mode: on the native tier an op that would leave this package's kernels raises instead."""
    global _STRICT
    _STRICT = bool(on)


def library_fallbacks(reset: bool = False) -> dict:
    out = dict(FALLBACKS)
    if reset:
        FALLBACKS.clear()
    return out


def _fallback(op: str, x: torch.Tensor, why: str = "") -> None:
    """Record (or, in strict mode, refuse) a non-native execution of ``op``; only CUDA tensors on the native tier
    count: CPU runs and the explicit library tier are not fallbacks."""
    if not (x.is_cuda and _TIER == "native"):
        return
    if _STRICT:
        raise RuntimeError(f"ops.{op}: no native kernel for this call ({why or 'unsupported shape / dtype'}); "
                           f"strict mode refuses the library / eager path")
    FALLBACKS[op] = FALLBACKS.get(op, 0) + 1


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and _TIER == "native"


def _nat():
    from . import native
    return native


# --------------------------------------------------------------------------- norms / elementwise
def rms_norm(x, weight, eps: float = 1e-6):
    if _native(x) and x.dtype == torch.bfloat16:
        return _nat().rms_norm(x, weight, eps)
    _fallback("rms_norm", x, str(x.dtype))
    return ref.rms_norm(x, weight, eps)


def layer_norm(x, weight=None, bias=None, eps: float = 1e-6):
    """LayerNorm over the last dim with optional affine.  Native tier: the LayerNorm-modulate kernel with
    ``scale = weight - 1`` and ``shift = bias`` (``LN(x) * (1 + scale) + shift``), rows flattened to one batch."""
    if _native(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _nat().layer_norm(x, weight, bias, eps)
    _fallback("layer_norm", x, f"{x.dtype} H={x.shape[-1]}")
    return ref.layer_norm(x, weight, bias, eps)


def layer_norm_modulate(x, scale, shift, eps: float = 1e-6):
    if _native(x) and x.dtype == torch.bfloat16:
        return _nat().layer_norm_modulate(x, scale, shift, eps)
    _fallback("layer_norm_modulate", x, str(x.dtype))
    return ref.layer_norm_modulate(x, scale, shift, eps)


def gated_residual(x, y, gate):
    if _native(x) and x.dtype == torch.bfloat16:
        return _nat().gated_residual(x, y, gate)
    _fallback("gated_residual", x, str(x.dtype))
    return ref.gated_residual(x, y, gate)


def swiglu(gate_up, clamp: Optional[float] = None):
    if _native(gate_up) and gate_up.dtype == torch.bfloat16 and clamp is None:
        return _nat().swiglu(gate_up)
    _fallback("swiglu", gate_up, "clamp" if clamp is not None else str(gate_up.dtype))
    return ref.swiglu(gate_up, clamp)


def gelu_tanh(x):
    if _native(x) and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
        return _nat().gelu(x, tanh=True)
    _fallback("gelu_tanh", x, str(x.dtype))
    return F.gelu(x, approximate="tanh")


def gelu(x):
    """Exact (erf) GELU."""
    if _native(x) and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
        return _nat().gelu(x, tanh=False)
    _fallback("gelu", x, str(x.dtype))
    return F.gelu(x)


def rope_rotate_half(x, cos, sin):
    if _native(x) and x.dtype == torch.bfloat16:
        return _nat().rope(x, cos, sin, interleaved=False)
    _fallback("rope_rotate_half", x, str(x.dtype))
    return ref.rope_rotate_half(x, cos, sin)


def rope_interleaved(x, cos, sin):
    if _native(x) and x.dtype == torch.bfloat16:
        return _nat().rope(x, cos, sin, interleaved=True)
    _fallback("rope_interleaved", x, str(x.dtype))
    return ref.rope_interleaved(x, cos, sin)


def l2_norm(x, eps: float = 1e-6):
    if _native(x) and x.dtype == torch.bfloat16 and x.shape[-1] <= 256:
        return _nat().l2_norm(x, eps)
    _fallback("l2_norm", x, f"{x.dtype} D={x.shape[-1]}")
    return ref.l2_norm(x, eps)


def gated_rms_norm(x, z, weight, eps: float = 1e-6):
    """``rmsnorm(x) * weight * silu(z)`` over the last dim, in ``z``'s dtype (``x`` may be the fp32 output of the delta rule)."""
    D = x.shape[-1]
    if (_native(x) and x.dtype in (torch.float32, torch.bfloat16) and z.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and D <= 256 and D % 8 == 0):
        return _nat().gated_rms_norm(x, z, weight, eps)
    _fallback("gated_rms_norm", x, f"x {x.dtype} z {z.dtype} D={D}")
    return ref.gated_rms_norm(x, z, weight, eps).to(z.dtype)


# --------------------------------------------------------------------------- GEMM
_RECOMPUTING = False


class recompute_region:
    """Marks the re-forward of a checkpointed unit (entered by the sharding engine's backward)."""

    def __enter__(self):
        global _RECOMPUTING
        self.prev, _RECOMPUTING = _RECOMPUTING, True

    def __exit__(self, *exc):
        global _RECOMPUTING
        _RECOMPUTING = self.prev


_ACT_CACHE = None      # (list, "record" | "replay") while a checkpointed unit runs under the sharding engine


class activation_cache:
    """Lets expensive, small-output ops (attention: out + log-sum-exp) keep their result across a checkpointed unit's
    first forward and its re-forward: ``record`` appends results to ``store``, ``replay`` hands them back in order.
    Same purpose as the reference's skip-recompute flash attention (fsdp/ops/flash_attn/skip_recompute_flash_attn.py:38,135)."""

    def __init__(self, store: list, mode: str):
        self.store, self.mode = store, mode

    def __enter__(self):
        global _ACT_CACHE
        self.prev, _ACT_CACHE = _ACT_CACHE, (self.store, self.mode)

    def __exit__(self, *exc):
        global _ACT_CACHE
        _ACT_CACHE = self.prev


def linear(x, weight, bias=None, value_unused_in_backward: bool = False):
    """``x @ weight.T + bias`` (weight is [out, in], K-major for both operands).

    ``value_unused_in_backward``: the caller promises that nothing downstream inside the checkpointed unit needs the
    VALUE of this product for its gradient (it only feeds a residual add).  During a recompute the native tier then
    skips the GEMM and returns an uninitialised tensor; gradients are unaffected."""
    if _native(x) and x.dtype == torch.bfloat16 and _nat().gemm_supported(x, weight):
        return _nat().linear(x, weight, bias, value_unused_in_backward and _RECOMPUTING)
    _fallback("linear", x, f"{x.dtype} {tuple(x.shape)} x {tuple(weight.shape)}")
    return F.linear(x, weight, bias)


def linear_swiglu(x, weight_gate_up):
    """``swiglu(x @ W_gate_up.T)``.  On the native tier a pass that keeps no graph (the first forward of a recomputed
    unit, inference) runs one kernel with the activation as the GEMM epilogue; a pass that will be differentiated keeps
    the pre-activation for the backward and runs GEMM and activation kernels."""
    if _native(x) and x.dtype == torch.bfloat16 and \
            not (torch.is_grad_enabled() and (x.requires_grad or weight_gate_up.requires_grad)) and \
            _nat().gemm_swiglu_supported(x, weight_gate_up):
        return _nat().gemm_swiglu(x, weight_gate_up)
    return swiglu(linear(x, weight_gate_up))


# --------------------------------------------------------------------------- attention
def attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int,
                     causal: bool = False, softmax_scale: Optional[float] = None):
    """Packed attention.  q: [T, Nq, D]; k, v: [T, Nkv, D]; cu_seqlens int32 on the same device."""
    if q.is_cuda:
        if _TIER == "native" and _nat().fmha_supported(q, k, v):
            return _nat().attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                           causal, softmax_scale, _ACT_CACHE)
        _fallback("attention_varlen", q, f"{q.dtype} D={q.shape[-1]}")
        return _library_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                         causal, softmax_scale)
    return ref.attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, softmax_scale)


def _library_attention_varlen(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale):
    from flash_attn import flash_attn_varlen_func
    D = q.shape[-1]
    pad = (-D) % 8
    if pad:  # flash-attn wants head_dim % 8 == 0 (ViT D=80 is fine; guard anyway)
        q, k, v = (F.pad(t, (0, pad)) for t in (q, k, v))
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = flash_attn_varlen_func(q, k, v, cu_q, cu_k, max_q, max_k, softmax_scale=scale, causal=causal)
    return out[..., :D] if pad else out


def attention_dense(q, k, v, causal: bool = False, softmax_scale: Optional[float] = None):
    """BSND attention (DiT).  q: [B, S, N, D]."""
    if q.is_cuda:
        B, Sq, N, D = q.shape
        Sk = k.shape[1]
        cq = torch.arange(0, (B + 1) * Sq, Sq, dtype=torch.int32, device=q.device)
        ck = torch.arange(0, (B + 1) * Sk, Sk, dtype=torch.int32, device=q.device)
        o = attention_varlen(q.reshape(B * Sq, N, D), k.reshape(B * Sk, -1, D), v.reshape(B * Sk, -1, D),
                             cq, ck, Sq, Sk, causal, softmax_scale)
        return o.view(B, Sq, N, D)
    return ref.attention_dense(q, k, v, causal, softmax_scale)


# --------------------------------------------------------------------------- loss
def linear_cross_entropy(h, weight, labels, ignore_index: int = -100, chunk: int = 2048):
    """Sum of token CE of ``h @ weight.T`` against ``labels`` without keeping [T, V] logits.

    Returns (loss_sum fp32 scalar, n_valid).  The library/CPU tier computes the loss and both
    gradients chunk by chunk inside forward (the reference does the same with
    ``torch.func.grad_and_value``: fsdp/features/memory/chunkloss/chunkloss.py:6-95).
    """
    if _native(h) and h.dtype == torch.bfloat16 and _nat().lce_supported(h, weight):
        return _nat().linear_cross_entropy(h, weight, labels, ignore_index)
    _fallback("linear_cross_entropy", h, str(h.dtype))
    return _ChunkedLinearCE.apply(h, weight, labels, ignore_index, chunk), (labels != ignore_index).sum()


class _ChunkedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, chunk):
        T = h.shape[0]
        dh = torch.empty_like(h)
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        loss = torch.zeros((), dtype=torch.float32, device=h.device)
        for s in range(0, T, chunk):
            hs = h[s:s + chunk]
            logits = (hs @ weight.t()).float()
            lab = labels[s:s + chunk]
            lse = torch.logsumexp(logits, -1)
            valid = lab != ignore_index
            safe = lab.clamp(min=0)
            tgt = logits.gather(1, safe[:, None]).squeeze(1)
            loss += ((lse - tgt) * valid).sum()
            p = torch.exp(logits - lse[:, None])
            p.scatter_add_(1, safe[:, None], -torch.ones_like(p[:, :1]))
            p *= valid[:, None]
            p = p.to(h.dtype)
            dh[s:s + chunk] = p @ weight
            dw += (p.t() @ hs).float()
        ctx.save_for_backward(dh, dw.to(weight.dtype))
        return loss

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        return dh * g.to(dh.dtype), dw * g.to(dw.dtype), None, None, None


# --------------------------------------------------------------------------- MoE
def grouped_gemm(x, w, counts):
    if _native(x) and x.dtype == torch.bfloat16 and _nat().grouped_gemm_supported(x, w):
        return _nat().grouped_gemm(x, w, counts)
    _fallback("grouped_gemm", x, str(x.dtype))
    return _GroupedGemmLoop.apply(x, w, counts)


class _GroupedGemmLoop(torch.autograd.Function):
    """Loop-of-matmuls grouped GEMM with explicit dgrad / wgrad (fsdp/ops/moe_ops/gemm.py:35-92)."""

    @staticmethod
    def forward(ctx, x, w, counts):
        ctx.save_for_backward(x, w)
        ctx.counts = [int(c) for c in counts]
        out = x.new_empty(x.shape[0], w.shape[-1])
        s = 0
        for e, c in enumerate(ctx.counts):
            if c:
                torch.matmul(x[s:s + c], w[e], out=out[s:s + c])
            s += c
        return out

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        dx = torch.empty_like(x)
        dw = torch.zeros_like(w)
        s = 0
        for e, c in enumerate(ctx.counts):
            if c:
                dx[s:s + c] = g[s:s + c] @ w[e].t()
                dw[e] = x[s:s + c].t() @ g[s:s + c]
            s += c
        return dx, dw, None


def moe_experts(tokens, topk_ids, probs, gate_up, down):
    """Local routed experts (all experts of ``gate_up`` / ``down`` live on this rank)."""
    if _native(tokens) and _nat().moe_supported(tokens, gate_up, down):
        return _nat().moe_experts(tokens, topk_ids, probs, gate_up, down)
    _fallback("moe_experts", tokens, str(tokens.dtype))
    permuted, order = ref.moe_permute(tokens, topk_ids)
    counts = torch.bincount(topk_ids.reshape(-1), minlength=gate_up.shape[0]).tolist()
    h = grouped_gemm(permuted, gate_up, counts)
    y = grouped_gemm(swiglu(h), down, counts)
    return ref.moe_unpermute(y, order, probs)


moe_permute = ref.moe_permute
moe_unpermute = ref.moe_unpermute

# --------------------------------------------------------------------------- GDN
def causal_conv1d(x, weight, bias=None, activation="silu", cu_seqlens=None):
    if _native(x) and bias is None and _nat().conv1d_supported(x, weight):
        return _nat().causal_conv1d(x, weight, activation, cu_seqlens)
    _fallback("causal_conv1d", x, "bias or unsupported shape")
    return ref.causal_conv1d(x, weight, bias, activation, cu_seqlens)


def gated_delta_rule(q, k, v, g, beta, scale=None, chunk: int = 64, initial_state=None):
    _fallback("gated_delta_rule", q, "batched form: use gated_delta_rule_varlen for the kernel path")
    return ref.gated_delta_rule_chunked(q, k, v, g, beta, scale, chunk, initial_state)


def gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, chunk: int = 64, scale=None):
    """Packed gated delta rule.  q, k: [T, H, K]; v: [T, H, V]; g, beta: [T, H]; the state restarts at every
    ``cu_seqlens`` boundary.  Returns [T, H, V] (fp32)."""
    if _native(q) and _nat().gdn_supported(q, v, chunk):
        return _nat().gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, chunk, scale)
    _fallback("gated_delta_rule_varlen", q, f"K={q.shape[-1]} V={v.shape[-1]} chunk={chunk}")
    outs = []
    cu = [int(c) for c in cu_seqlens]
    for a, b in zip(cu[:-1], cu[1:]):
        o, _ = ref.gated_delta_rule_chunked(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b], beta[None, a:b], scale, chunk)
        outs.append(o[0])
    return torch.cat(outs, 0)


def kda(q, k, v, g, beta, scale=None, chunk: int = 64, initial_state=None):
    """Kimi delta attention (per-channel gate) on [B, T, H, *] tensors.  Returns (o fp32, final state)."""
    if initial_state is None and chunk == 64 and _native(q) and _nat().gdn_supported(q[0], v[0], chunk):
        B, T = q.shape[:2]
        cu = [i * T for i in range(B + 1)]
        flat = lambda t: t.reshape((B * T,) + tuple(t.shape[2:]))
        o = kda_varlen(flat(q), flat(k), flat(v), flat(g), flat(beta), cu, scale)
        return o.view(B, T, *o.shape[1:]).float(), None
    _fallback("kda", q, f"K={q.shape[-1]} V={v.shape[-1]} chunk={chunk} initial_state={initial_state is not None}")
    return ref.kda_chunked(q, k, v, g, beta, scale, chunk, initial_state)


def kda_varlen(q, k, v, g, beta, cu_seqlens, scale=None):
    """Kimi delta attention on packed sequences: q, k, g [T, H, K], v [T, H, V], beta [T, H]; the state restarts at every
    ``cu_seqlens`` boundary.  On CUDA (K = V = 128) the state walk is the tcgen05 kernel with one decay per key channel;
    elsewhere the same chunked form runs in PyTorch."""
    from . import gdn
    if not (_native(q) and _nat().gdn_supported(q, v, 64)):
        _fallback("kda_varlen", q, f"K={q.shape[-1]} V={v.shape[-1]}")
        if q.is_cuda:            # the autograd function would pick the kernel for a shape it does not support
            outs = []
            cu = [int(c) for c in cu_seqlens]
            for a, b in zip(cu[:-1], cu[1:]):
                outs.append(ref.kda_chunked(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b], beta[None, a:b], scale)[0][0])
            return torch.cat(outs, 0).to(v.dtype)
    return gdn.kimi_delta_attention_varlen(q, k, v, g, beta, cu_seqlens, scale)


def status() -> dict:
    """Which ops have a native sm_100a implementation loaded (for logs and DESIGN tables)."""
    try:
        return _nat().status()
    except Exception as e:  # extension absent on a CPU box
        return {"loaded": False, "why": str(e)}


class LayerNorm(torch.nn.LayerNorm):
    """``torch.nn.LayerNorm`` (same parameters and state-dict keys) whose forward goes through :func:`layer_norm`,
    i.e. the LayerNorm kernel of this package on the native tier."""

    def forward(self, x):
        if len(self.normalized_shape) != 1:
            return super().forward(x)
        return layer_norm(x, self.weight, self.bias, self.eps)


if os.environ.get("MM_B200_SANITIZE", "") not in ("", "0"):
    from . import sanitize as _sanitize
    _sanitize.enable()
