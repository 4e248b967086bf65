"""ctypes bindings and autograd wrappers for the sm_100a kernels in ``csrc/``.

The library is loaded from ``ops/_lib/libmm_b200_ops.so`` (built in-tree by ``ops/build.py``).  On a
GPU box a missing or stale library is an error, never a silent fallback.  Kernels take raw device
pointers and the current CUDA stream; tensors are kept alive by the autograd contexts / callers.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

from . import build as _build

_LIB = None
_STATUS: dict = {}
# forward attention kernel: 3 = split softmax, O accumulated in tensor memory with lazy rescaling
# (csrc/fmha_fwd_split.cuh, default); 0 = one softmax warpgroup, O folded in registers (csrc/fmha_fwd.cu, fallback)
FMHA_FWD_VARIANT = int(os.environ.get("MM_B200_FMHA_FWD_VARIANT", "3"))
LAUNCHES = 0  # native kernel launches issued through this module (bench reports it)

_p, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float


def lib():
    global _LIB
    if _LIB is None:
        path = _build.lib_path()
        if not os.path.exists(path):
            raise RuntimeError(f"native op library not built: {path} (run python -m mindspeed_mm_b200.ops.build)")
        _LIB = C.CDLL(path)
        _declare(_LIB)
        _LIB.mm_fmha_set_fwd_variant(FMHA_FWD_VARIANT)
    return _LIB


# Row norms: rows of up to 256 elements (per-head q/k norms, L2 norm of GDN heads) take a lane group per row
# (csrc/rownorm.cu: 0.94 of the copy bandwidth against 0.45 for a block per row); longer rows keep a block per row
# (csrc/elementwise.cu), which measured faster there (0.67 against 0.45 at 3584).
def _row_group(H: int) -> bool:
    return H <= 256 and H % 8 == 0


def _declare(L):
    sig = {
        "mm_rmsnorm_fwd": [_p, _p, _p, _p, _i, _i, _f, _p],
        "mm_rownorm_rms_fwd": [_p, _p, _p, _p, _ll, _i, _f, _p],
        "mm_rownorm_ln_mod_fwd": [_p, _p, _p, _p, _p, _p, _ll, _i, _i, _f, _p],
        "mm_rownorm_l2_fwd": [_p, _p, _p, _ll, _i, _f, _p],
        "mm_gated_rms_fwd": [_p, _i, _p, _p, _p, _p, _ll, _i, _f, _p],
        "mm_gated_rms_bwd": [_p, _i, _p, _p, _p, _p, _p, _p, _p, _ll, _i, _p],
        "mm_rmsnorm_bwd_grid": [_i],
        "mm_sq_norm_blocks": [],
        "mm_rmsnorm_set_v16": [_i],
        "mm_sq_norm": [_p, _ll, _p, _p],
        "mm_rmsnorm_bwd": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _p],
        "mm_swiglu_fwd": [_p, _p, _ll, _i, _p],
        "mm_swiglu_bwd": [_p, _p, _p, _ll, _i, _p],
        "mm_gelu_fwd": [_p, _p, _ll, _i, _p],
        "mm_gelu_bwd": [_p, _p, _p, _ll, _i, _p],
        "mm_rope_half": [_p, _ll, _p, _p, _p, _i, _i, _i, _i, _p],
        "mm_rope_interleaved": [_p, _ll, _p, _p, _p, _i, _i, _i, _i, _p],
        "mm_ln_mod_fwd": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _f, _p],
        "mm_ln_mod_bwd_ctas": [_i, _i],
        "mm_ln_mod_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p],
        "mm_gated_residual": [_p, _p, _p, _p, _ll, _i, _i, _p],
        "mm_adamw": [_p, _p, _p, _p, _i, _p, _ll, _ll, _f, _f, _f, _f, _f, _f, _f, _f, _p, _p],
        "mm_gemm_bf16": [_p, _p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _p, _p],
        "mm_gemm_swiglu_bf16": [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _p, _p],
        "mm_ce_fwd_bwd": [_p, _ll, _p, _p, _i, _i, _i, _p],
        "mm_fmha_max_tiles": [_i, _i],
        "mm_fmha_set_fwd_variant": [_i],
        "mm_fmha_fwd": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _i, _f, _p, _p],
        "mm_fmha_bwd_max_tiles": [_i, _i],
        "mm_fmha_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _i, _f,
                        _i, _i, _p, _p],
        "mm_grouped_gemm_max_tiles": [_i, _i, _i, _i, _i],
        "mm_grouped_gemm_bf16": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _p],
        "mm_moe_permute": [_p, _p, _p, _i, _i, _p],
        "mm_moe_unpermute": [_p, _p, _p, _p, _i, _i, _i, _p],
        "mm_conv1d_fwd": [_p, _p, _p, _p, _i, _i, _i, _i, _p],
        "mm_conv1d_bwd": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p],
        "mm_l2norm_fwd": [_p, _p, _p, _ll, _i, _f, _p],
        "mm_l2norm_bwd": [_p, _p, _p, _p, _ll, _i, _p],
        "mm_gdn_prologue": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _f, _p],
        "mm_gdn_fwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p],
        "mm_gdn_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p],
        "mm_p2p_scatter_rows": [_p, _p, _p, _p, _p, _i, _i, _i, _p],
        "mm_p2p_gather_rows": [_p, _p, _p, _p, _i, _i, _i, _p],
        "mm_p2p_copy": [_p, _p, _ll, _i, _p],
        "mm_p2p_set_wait_limit": [_ll],
        "mm_p2p_flag_bytes": [],
        "mm_p2p_allgather": [_p, _p, _ll, _i, _i, _i, _p],
        "mm_p2p_allgather_ce": [_p, _p, _ll, _i, _i, _p],
        "mm_p2p_rs_adamw": [_p, _p, _ll, _i, _i, _i, C.c_uint, _f, _p, _p, _p, _p, _ll, _f, _f, _f, _f, _f, _f, _f,
                            _p, _i, _p],
        "mm_p2p_rs": [_p, _p, _ll, _i, _i, _i, C.c_uint, _f, _p, _i, _p, _i, _p],
        "mm_p2p_wait_done": [_p, _i, C.c_uint, _i, _i, _p, _p],
        "mm_p2p_barrier_bytes": [],
        "mm_p2p_barrier": [_p, _i, _i, C.c_uint, _p, _p],
    }
    for name, args in sig.items():
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = _i
            _STATUS[name] = True
        else:
            _STATUS[name] = False


def status() -> dict:
    lib()
    return {"loaded": True, "path": _build.lib_path(), "symbols": dict(_STATUS)}


def _st():
    return torch.cuda.current_stream().cuda_stream


def _eager(op: str, x, why: str):
    """An op of this module was called with a shape its kernel does not take: count it (or refuse, in strict mode)
    through the front end's fallback register, then let the caller run the PyTorch form."""
    from .. import ops as _ops
    _ops._fallback(op, x, why)


SYNC_CHECK = False   # ops/sanitize.py: synchronise after every native call and read the status word, so that an
                     # asynchronous error is reported under the name of the op that launched it


def _check(rc: int, what: str):
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
    if SYNC_CHECK and torch.cuda.is_available():
        try:
            torch.cuda.synchronize()
        except RuntimeError as e:
            raise RuntimeError(f"{what}: device error surfaced after this launch: {e}") from e
        for key, word in _status_words.items():
            v = int(word.item())
            if v:
                word.zero_()
                raise RuntimeError(f"{what}: a bounded wait ran out on device {key} (status {v})")


_status_words: dict = {}


def status_word(device) -> torch.Tensor:
    """Device int the tcgen05 kernels write when a bounded wait ran out (0 = fine)."""
    key = torch.device(device).index or 0
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def check_status(device=None) -> int:
    """Host-side read of the status word (synchronises); raises if a kernel reported a timeout."""
    dev = device if device is not None else torch.cuda.current_device()
    v = int(status_word(dev).item())
    if v != 0:
        status_word(dev).zero_()
        raise RuntimeError(f"a native kernel gave up a bounded wait (status {v})")
    return v


# --------------------------------------------------------------------------- RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        wc = w.contiguous()
        fn = lib().mm_rownorm_rms_fwd if _row_group(H) else lib().mm_rmsnorm_fwd
        _check(fn(x2.data_ptr(), wc.data_ptr(), y.data_ptr(), rstd.data_ptr(), T, H, eps, _st()), "rmsnorm_fwd")
        ctx.save_for_backward(x2, wc, rstd)
        ctx.shape = shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        T, H = x2.shape
        dy2 = dy.reshape(T, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        grid = lib().mm_rmsnorm_bwd_grid(T)
        partial = torch.empty(grid * H, dtype=torch.float32, device=x2.device)
        _check(lib().mm_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                    dw.data_ptr(), partial.data_ptr(), T, H, _st()), "rmsnorm_bwd")
        return dx.view(ctx.shape), dw, None


def rms_norm(x, w, eps=1e-6):
    if x.shape[-1] % 8 or x.shape[-1] > 8192:
        from . import reference
        _eager("rms_norm", x, f"H={x.shape[-1]}")
        return reference.rms_norm(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


# --------------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        T, F = g2.shape[0], F2 // 2
        out = torch.empty(T, F, dtype=gu.dtype, device=gu.device)
        _check(lib().mm_swiglu_fwd(g2.data_ptr(), out.data_ptr(), T, F, _st()), "swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        T, F = g2.shape[0], g2.shape[1] // 2
        d2 = dout.reshape(T, F)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        din = torch.empty_like(g2)
        _check(lib().mm_swiglu_bwd(g2.data_ptr(), d2.data_ptr(), din.data_ptr(), T, F, _st()), "swiglu_bwd")
        return din.view(ctx.shape)


def swiglu(gu):
    if (gu.shape[-1] // 2) % 8:
        from . import reference
        _eager("swiglu", gu, f"F={gu.shape[-1] // 2}")
        return reference.swiglu(gu)
    return _SwiGLU.apply(gu)


# --------------------------------------------------------------------------- RoPE
class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tanh):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _check(lib().mm_gelu_fwd(xc.data_ptr(), y.data_ptr(), xc.numel(), int(tanh), _st()), "gelu_fwd")
        ctx.save_for_backward(xc)
        ctx.tanh = tanh
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(x)
        _check(lib().mm_gelu_bwd(x.data_ptr(), dyc.data_ptr(), dx.data_ptr(), x.numel(), int(ctx.tanh), _st()), "gelu_bwd")
        return dx.view(dy.shape), None


def gelu(x, tanh: bool = True):
    """bf16 GELU (tanh approximation or exact erf form); element count a multiple of 8."""
    return _Gelu.apply(x, bool(tanh))


def _rope_call(x, cos, sin, interleaved, backward):
    # x: [T, N, D] whose last two dims are dense; the token stride may be larger (view into fused qkv)
    T, N, D = x.shape
    if x.stride(2) != 1 or x.stride(1) != D or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    out = torch.empty(T, N, D, dtype=x.dtype, device=x.device)
    if interleaved:
        _check(lib().mm_rope_interleaved(x.data_ptr(), x.stride(0), cos.data_ptr(), sin.data_ptr(), out.data_ptr(),
                                         T, N, D, int(backward), _st()), "rope_interleaved")
    else:
        _check(lib().mm_rope_half(x.data_ptr(), x.stride(0), cos.data_ptr(), sin.data_ptr(), out.data_ptr(),
                                  T, N, D, int(backward), _st()), "rope_half")
    return out


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, interleaved):
        ctx.save_for_backward(cos, sin)
        ctx.interleaved = interleaved
        return _rope_call(x, cos, sin, interleaved, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _rope_call(dy, cos, sin, ctx.interleaved, True), None, None, None


def rope(x, cos, sin, interleaved: bool):
    T, N, D = x.shape
    if interleaved:
        if D % 8:
            from . import reference
            _eager("rope_interleaved", x, f"D={D}")
            return reference.rope_interleaved(x, cos, sin)
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
    else:
        if D % 8:
            from . import reference
            _eager("rope_rotate_half", x, f"D={D}")
            return reference.rope_rotate_half(x, cos, sin)
        cos, sin = cos.to(torch.bfloat16).contiguous(), sin.to(torch.bfloat16).contiguous()
    return _Rope.apply(x, cos, sin, interleaved)


# --------------------------------------------------------------------------- adaLN
class _LNMod(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift, eps):
        B, S, H = x.shape
        xc, sc, sh = x.contiguous(), scale.reshape(B, H).contiguous(), shift.reshape(B, H).contiguous()
        y = torch.empty_like(xc)
        mean = torch.empty(B * S, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        fn = lib().mm_rownorm_ln_mod_fwd if _row_group(H) else lib().mm_ln_mod_fwd
        _check(fn(xc.data_ptr(), sc.data_ptr(), sh.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), B * S, S, H,
                  eps, _st()), "ln_mod_fwd")
        ctx.save_for_backward(xc, sc, mean, rstd)
        ctx.sshape = scale.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x, sc, mean, rstd = ctx.saved_tensors
        B, S, H = x.shape
        dyc = dy.contiguous()
        dx = torch.empty_like(x)
        dscale = torch.empty_like(sc)
        dshift = torch.empty_like(sc)
        per = lib().mm_ln_mod_bwd_ctas(B, S)
        partial = torch.empty(2 * B * per * H, dtype=torch.float32, device=x.device)
        _check(lib().mm_ln_mod_bwd(x.data_ptr(), sc.data_ptr(), dyc.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                   dx.data_ptr(), dscale.data_ptr(), dshift.data_ptr(), partial.data_ptr(), B, S, H,
                                   _st()), "ln_mod_bwd")
        return dx, dscale.view(ctx.sshape), dshift.view(ctx.sshape), None


def layer_norm_modulate(x, scale, shift, eps=1e-6):
    """x: [B, S, H]; scale/shift: [B, 1, H] or [B, H]."""
    if x.dim() != 3 or x.shape[-1] % 8 or x.shape[-1] > 8192 or scale.numel() != x.shape[0] * x.shape[-1]:
        from . import reference
        _eager("layer_norm_modulate", x, f"x {tuple(x.shape)} scale {tuple(scale.shape)}")
        return reference.layer_norm_modulate(x, scale, shift, eps)
    return _LNMod.apply(x, scale.to(x.dtype), shift.to(x.dtype), eps)


def layer_norm(x, weight=None, bias=None, eps=1e-6):
    """LayerNorm over the last dim of a bf16 tensor through the LayerNorm-modulate kernels: all rows form one batch,
    ``scale = weight - 1`` and ``shift = bias`` (zeros when absent), so ``LN(x) * (1 + scale) + shift`` is the affine
    LayerNorm.  Gradients of weight / bias come out of the kernel's per-batch scale / shift reductions."""
    H = x.shape[-1]
    if weight is not None:
        scale = (weight.float() - 1.0).to(x.dtype).view(1, H)
    else:
        scale = torch.zeros(1, H, dtype=x.dtype, device=x.device)
    shift = bias.to(x.dtype).view(1, H) if bias is not None else torch.zeros(1, H, dtype=x.dtype, device=x.device)
    return _LNMod.apply(x.reshape(1, -1, H), scale, shift, eps).view(x.shape)


class _GatedResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, gate):
        B, S, H = x.shape
        xc, yc, gc = x.contiguous(), y.contiguous(), gate.reshape(B, H).contiguous()
        out = torch.empty_like(xc)
        _check(lib().mm_gated_residual(xc.data_ptr(), yc.data_ptr(), gc.data_ptr(), out.data_ptr(), B * S, S, H,
                                       _st()), "gated_residual")
        ctx.save_for_backward(yc, gc)
        ctx.gshape = gate.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        y, g = ctx.saved_tensors
        B, S, H = y.shape
        dy = dout * g.view(B, 1, H)
        dg = (dout.float() * y.float()).sum(1).to(g.dtype).view(ctx.gshape)
        return dout, dy, dg


def gated_residual(x, y, gate):
    if x.dim() != 3 or x.shape[-1] % 8 or gate.numel() != x.shape[0] * x.shape[-1]:
        from . import reference
        _eager("gated_residual", x, f"x {tuple(x.shape)} gate {tuple(gate.shape)}")
        return reference.gated_residual(x, y, gate)
    return _GatedResidual.apply(x, y, gate.to(x.dtype))


# --------------------------------------------------------------------------- AdamW
def sq_norm(tensors) -> torch.Tensor:
    """Sum of squares over a list of fp32 CUDA tensors (the squared global gradient norm of flat shards): one launch per
    tensor into a fixed-order table of block partials, one reduction at the end."""
    nb = lib().mm_sq_norm_blocks()
    partials = torch.zeros(len(tensors), nb, dtype=torch.float32, device=tensors[0].device)
    st = _st()
    for i, t in enumerate(tensors):
        t = t.contiguous()
        if t.data_ptr() % 16:           # a view at an odd offset: the kernel reads 16-byte vectors
            t = t.clone()
        _check(lib().mm_sq_norm(t.data_ptr(), t.numel(), partials[i].data_ptr(), st), "sq_norm")
    return partials.sum()


def adamw_shard(master, exp_avg, exp_avg_sq, grad, p16, lr, b1, b2, eps, wd, step, split, grad_scale=1.0):
    n = master.numel()
    scale_ptr = None
    gs = 1.0
    if isinstance(grad_scale, torch.Tensor):
        scale_ptr = grad_scale.float().reshape(1)
        sp = scale_ptr.data_ptr()
    else:
        gs = float(grad_scale)
        sp = None
    bc1 = 1.0 - b1 ** step
    bc2 = 1.0 - b2 ** step
    g = grad if grad.dtype in (torch.bfloat16, torch.float32) else grad.float()
    _check(lib().mm_adamw(master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), g.data_ptr(),
                          int(g.dtype == torch.bfloat16), p16.data_ptr(), n, int(split), lr, b1, b2, eps, wd, bc1, bc2,
                          gs, sp, _st()), "adamw")


# --------------------------------------------------------------------------- GEMM (tcgen05)
def _gemm_raw(a, b, out, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, bn=None):
    if bn is None:
        bn = 256 if N >= 256 else 128
    st = status_word(a.device)
    rc = lib().mm_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), None if bias is None else bias.data_ptr(),
                            M, N, K, lda, ldb, ldc, int(a_mn), int(b_mn), bn, st.data_ptr(), _st())
    _check(rc, "gemm_bf16")


def _ok2d(t):
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def gemm_supported(x, w) -> bool:
    return (os.environ.get("MM_B200_GEMM", "1") == "1" and w.dtype == torch.bfloat16 and w.dim() == 2
            and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0)


def gemm_nt(a, b, bias=None, out=None):
    """a [M,K] @ b[N,K]^T (+bias) -> [M,N]."""
    if not _ok2d(a):
        a = a.contiguous()
    if not _ok2d(b):
        b = b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    _gemm_raw(a, b, out, bias, M, N, K, a.stride(0), b.stride(0), out.stride(0), 0, 0)
    return out


def gemm_swiglu_supported(x, w) -> bool:
    return gemm_supported(x, w) and w.shape[0] % 256 == 0 and os.environ.get("MM_B200_GEMM_SWIGLU", "1") == "1"


def gemm_swiglu(x, w):
    """``silu(x W_gate^T) * (x W_up^T)`` for the fused ``w = [W_gate; W_up]`` ([2F, K]) in one kernel: the activation is the
    GEMM epilogue and the [T, 2F] pre-activation is never written.  No autograd: for passes that keep no graph."""
    shape = x.shape
    a = x.reshape(-1, shape[-1])
    if not _ok2d(a):
        a = a.contiguous()
    if not _ok2d(w):
        w = w.contiguous()
    M, K = a.shape
    F = w.shape[0] // 2
    out = torch.empty(M, F, dtype=torch.bfloat16, device=a.device)
    st = status_word(a.device)
    _check(lib().mm_gemm_swiglu_bf16(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, F, K, a.stride(0), w.stride(0),
                                     out.stride(0), st.data_ptr(), _st()), "gemm_swiglu_bf16")
    return out.view(*shape[:-1], F)


def gemm_nn(a, b, out=None):
    """a [M,K] @ b[K,N] -> [M,N]  (b read N-contiguous: dgrad)."""
    if not _ok2d(a):
        a = a.contiguous()
    if not _ok2d(b):
        b = b.contiguous()
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    _gemm_raw(a, b, out, None, M, N, K, a.stride(0), b.stride(0), out.stride(0), 0, 1)
    return out


def gemm_tn(a, b, out=None):
    """a[K,M]^T @ b[K,N] -> [M,N]  (both read with the contraction dim strided: wgrad)."""
    if not _ok2d(a):
        a = a.contiguous()
    if not _ok2d(b):
        b = b.contiguous()
    K, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    _gemm_raw(a, b, out, None, M, N, K, a.stride(0), b.stride(0), out.stride(0), 1, 1)
    return out


_BWD_NATIVE = os.environ.get("MM_B200_GEMM_BWD", "1") == "1"


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, skip_value=False):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.shape = shape
        if skip_value:
            # re-forward of a checkpointed unit whose last linear feeds only a residual add: the gradient needs the
            # operands, not the product, so the GEMM is not run again
            return torch.empty(*shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
        y = gemm_nt(x2, w, bias)
        return y.view(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = (gemm_nn(dy2, w) if _BWD_NATIVE else dy2 @ w).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            tgt = getattr(w, "_grad_flat", None)
            if tgt is not None and _BWD_NATIVE and w.grad is None:
                # the sharding engine offered this parameter's slice of the unit's flat gradient buffer: write the
                # weight gradient there (a fresh view each time, so autograd can adopt it as .grad without a copy)
                flat, off, numel, shape = tgt
                w._grad_flat = None                      # a second use of the same weight falls back to a new tensor
                dw = gemm_tn(dy2, x2, out=flat[off:off + numel].view(shape))
            else:
                dw = gemm_tn(dy2, x2) if _BWD_NATIVE else dy2.t() @ x2
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = torch.sum(dy2, 0, dtype=torch.float32).to(dy2.dtype)
        return dx, dw, db, None


def linear(x, w, bias=None, skip_value=False):
    return _Linear.apply(x, w, bias, skip_value)


# --------------------------------------------------------------------------- not yet native
def fmha_supported(q, k, v) -> bool:
    """bf16, one head dim for q / k / v, at most 128 and a multiple of 8 (the kernels work on 128-wide tiles; a narrower
    head, e.g. the vision tower's 80, is zero-filled by the TMA loads, not padded in memory), GQA groups whole."""
    D = q.shape[-1]
    return (os.environ.get("MM_B200_FMHA", "1") == "1" and q.dtype == torch.bfloat16 and D <= 128 and D % 8 == 0
            and k.shape[-1] == D and v.shape[-1] == D and q.shape[1] % k.shape[1] == 0)


def _dense_heads(t):
    """[T, N, D] with unit stride on D, D between heads and an 8-element aligned token stride (views into a
    fused qkv tensor qualify); anything else is copied."""
    T, N, D = t.shape
    if t.stride(2) != 1 or t.stride(1) != D or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def fmha_forward(q, k, v, cu_q, cu_k, causal, scale):
    """Returns (out [T, Nq, D] bf16, lse [Nq, T] fp32) from the tcgen05 kernel."""
    q, k, v = _dense_heads(q), _dense_heads(k), _dense_heads(v)
    T, Nq, D = q.shape
    Tk, Nkv = k.shape[0], k.shape[1]
    n_seqs = cu_q.numel() - 1
    out = torch.empty(T, Nq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(Nq, T, dtype=torch.float32, device=q.device)
    plan = torch.empty(3 * lib().mm_fmha_max_tiles(T, n_seqs) + 1, dtype=torch.int32, device=q.device)
    cu_q = cu_q.to(torch.int32)
    cu_k = cu_k.to(torch.int32)
    rc = lib().mm_fmha_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), cu_q.data_ptr(),
                           cu_k.data_ptr(), plan.data_ptr(), T, Tk, n_seqs, Nq, Nkv, D, q.stride(0), k.stride(0),
                           v.stride(0), int(causal), float(scale), status_word(q.device).data_ptr(), _st())
    _check(rc, "fmha_fwd")
    return out, lse


# backward kernels: dQ kernel + dK/dV kernel over 128-row query steps (5, default) or over 64-row steps (0, fallback)
FMHA_BWD_VARIANT = int(os.environ.get("MM_B200_FMHA_BWD_VARIANT", "5"))
FMHA_BWD = os.environ.get("MM_B200_FMHA_BWD", "native")     # "native" (tcgen05 kernels) or "flash" (flash-attn library)


def fmha_backward(do, q, k, v, out, lse, cu_q, cu_k, causal, scale):
    """dq, dk, dv from the tcgen05 backward kernels (dQ kernel + dK/dV kernel, no atomics)."""
    q, k, v = _dense_heads(q), _dense_heads(k), _dense_heads(v)
    do, out = do.contiguous(), out.contiguous()
    T, Nq, D = q.shape
    Tk, Nkv = k.shape[0], k.shape[1]
    n_seqs = cu_q.numel() - 1
    dev = q.device
    dq = torch.empty(T, Nq, D, dtype=q.dtype, device=dev)
    # GQA: one dK/dV CTA per QUERY head (more, shorter CTAs); the group's partials are summed afterwards
    split = Nq != Nkv
    dk = torch.empty(Tk, Nq if split else Nkv, D, dtype=q.dtype, device=dev)
    dv = torch.empty(Tk, Nq if split else Nkv, D, dtype=q.dtype, device=dev)
    delta = torch.empty(Nq, T, dtype=torch.float32, device=dev)
    L = lib()
    plan = torch.empty(3 * (L.mm_fmha_bwd_max_tiles(T, n_seqs) + L.mm_fmha_bwd_max_tiles(Tk, n_seqs)) + 2,
                       dtype=torch.int32, device=dev)
    cu_q, cu_k = cu_q.to(torch.int32), cu_k.to(torch.int32)
    rc = L.mm_fmha_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(),
                       delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu_q.data_ptr(), cu_k.data_ptr(),
                       plan.data_ptr(), T, Tk, n_seqs, Nq, Nkv, D, q.stride(0), k.stride(0), v.stride(0), int(causal),
                       float(scale), int(split), FMHA_BWD_VARIANT, status_word(dev).data_ptr(), _st())
    _check(rc, "fmha_bwd")
    global LAUNCHES
    LAUNCHES += 4
    if split:
        G = Nq // Nkv
        dk = torch.sum(dk.view(Tk, Nkv, G, D), 2, dtype=torch.float32).to(q.dtype)
        dv = torch.sum(dv.view(Tk, Nkv, G, D), 2, dtype=torch.float32).to(q.dtype)
    return dq, dk, dv


class _FMHA(torch.autograd.Function):
    """Forward and backward: tcgen05 kernels (``MM_B200_FMHA_BWD=flash`` switches the backward to flash-attn's
    varlen backward fed with this forward's out / lse, for comparison)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, precomputed=None):
        out, lse = precomputed if precomputed is not None else fmha_forward(q, k, v, cu_q, cu_k, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.meta = (max_q, max_k, causal, scale)
        ctx.lse_out = lse
        return out

    @staticmethod
    def backward(ctx, do):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, causal, scale = ctx.meta
        if FMHA_BWD == "native" and _STATUS.get("mm_fmha_bwd", False):
            dq, dk, dv = fmha_backward(do, q, k, v, out, lse, cu_q, cu_k, causal, scale)
            return dq, dk, dv, None, None, None, None, None, None, None
        dq, dk, dv = torch.empty(q.shape, dtype=q.dtype, device=q.device), torch.empty(k.shape, dtype=k.dtype, device=k.device), \
            torch.empty(v.shape, dtype=v.dtype, device=v.device)
        _flash_attn_varlen_backward(do.contiguous(), q, k, v, out, lse, dq, dk, dv, cu_q.to(torch.int32), cu_k.to(torch.int32),
                                    max_q, max_k, 0.0, scale, causal, -1, -1, 0.0, None, False)
        return dq, dk, dv, None, None, None, None, None, None, None


def attention_varlen(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, cache=None):
    """``cache`` = (store, mode) from :class:`ops.activation_cache`: under ``record`` (the no-grad first forward of a
    checkpointed unit) the output and log-sum-exp are kept, under ``replay`` (its re-forward) they are reused and the
    forward kernel is not run again."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if cache is not None:
        store, mode = cache
        if mode == "record" and not torch.is_grad_enabled():
            out, lse = fmha_forward(q, k, v, cu_q, cu_k, bool(causal), float(scale))
            store.append((out, lse))
            return out
        if mode == "replay" and store:
            return _FMHA.apply(q, k, v, cu_q, cu_k, max_q, max_k, bool(causal), float(scale), store.pop(0))
    return _FMHA.apply(q, k, v, cu_q, cu_k, max_q, max_k, bool(causal), float(scale))


def lce_supported(h, w) -> bool:
    return gemm_supported(h, w) and h.dim() == 2


class _LinearCE(torch.autograd.Function):
    """loss_sum = sum_t CE(h_t W^T, label_t).  Forward already produces both gradients:
    logits GEMM (tcgen05) -> in-place softmax-minus-onehot kernel -> dgrad and wgrad GEMMs (tcgen05);
    backward only scales them by the incoming scalar.  Rows are processed in chunks so that the bf16
    logits buffer stays a bounded slab (the reference chunks for the same reason:
    fsdp/features/memory/chunkloss/chunkloss.py:6-95)."""

    @staticmethod
    def forward(ctx, h, w, labels, ignore_index, chunk):
        T, H = h.shape
        V = w.shape[0]
        h = h.contiguous()
        labels = labels.contiguous()
        row_loss = torch.empty(T, dtype=torch.float32, device=h.device)
        dh = torch.empty_like(h)
        dw = torch.empty_like(w)
        chunk = min(chunk, T)
        logits = torch.empty(chunk, V, dtype=torch.bfloat16, device=h.device)
        dw_acc = None
        n_chunks = (T + chunk - 1) // chunk
        for c in range(n_chunks):
            a, b = c * chunk, min(T, (c + 1) * chunk)
            z = logits[: b - a]
            gemm_nt(h[a:b], w, out=z)
            _check(lib().mm_ce_fwd_bwd(z.data_ptr(), z.stride(0), labels[a:b].data_ptr(), row_loss[a:b].data_ptr(),
                                       b - a, V, ignore_index, _st()), "ce_fwd_bwd")
            gemm_nn(z, w, out=dh[a:b])
            if n_chunks == 1:
                gemm_tn(z, h[a:b], out=dw)
            else:
                part = gemm_tn(z, h[a:b])
                dw_acc = part.float() if dw_acc is None else dw_acc.add_(part)
        if dw_acc is not None:
            dw.copy_(dw_acc)
        ctx.save_for_backward(dh, dw)
        return row_loss.sum()

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        gs = g.to(dh.dtype)
        return dh.mul_(gs), dw.mul_(gs), None, None, None


def linear_cross_entropy(h, w, labels, ignore_index=-100, chunk=8192):
    loss = _LinearCE.apply(h, w, labels, ignore_index, chunk)
    return loss, (labels != ignore_index).sum()


def grouped_gemm_supported(x, w) -> bool:
    return False      # the native MoE path works on the aligned layout: see moe_experts()


# --------------------------------------------------------------------------- MoE on the aligned layout
def moe_supported(tokens, gate_up, down) -> bool:
    return (os.environ.get("MM_B200_MOE", "1") == "1" and tokens.dtype == torch.bfloat16 and tokens.shape[-1] % 128 == 0
            and gate_up.shape[-1] % 256 == 0 and down.shape[-1] % 128 == 0)


def aligned_routing(topk_ids, num_experts: int):
    """Device-side plan of the aligned expert-major layout (no host sync): every expert's rows start at a
    multiple of 128.  Returns (off [E+1] int32, row_of_pair [T*k] int32, src_of_row [R] int32 (-1 = pad), R)."""
    T, k = topk_ids.shape
    flat = topk_ids.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + 127) // 128 * 128
    off = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    off[1:] = padded.cumsum(0)
    ustart = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    ustart[1:] = counts.cumsum(0)
    sorted_e = flat[order]
    rows = off[sorted_e] + (torch.arange(flat.numel(), device=flat.device) - ustart[sorted_e])
    R = (T * k + num_experts * 127 + 127) // 128 * 128            # static upper bound of off[E]
    row_of_pair = torch.empty(T * k, dtype=torch.int32, device=flat.device)
    row_of_pair[order] = rows.to(torch.int32)
    src_of_row = torch.full((R,), -1, dtype=torch.int32, device=flat.device)
    src_of_row[rows] = (order // k).to(torch.int32)
    return off.to(torch.int32), row_of_pair, src_of_row, R


class _AlignedPermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, src_of_row, row_of_pair, k):
        R, H = src_of_row.numel(), tokens.shape[1]
        out = torch.empty(R, H, dtype=tokens.dtype, device=tokens.device)
        _check(lib().mm_moe_permute(tokens.contiguous().data_ptr(), src_of_row.data_ptr(), out.data_ptr(), R, H, _st()),
               "moe_permute")
        ctx.save_for_backward(row_of_pair)
        ctx.k, ctx.T = k, tokens.shape[0]
        return out

    @staticmethod
    def backward(ctx, g):
        (row_of_pair,) = ctx.saved_tensors
        ones = torch.ones(ctx.T * ctx.k, dtype=g.dtype, device=g.device)
        out = torch.empty(ctx.T, g.shape[1], dtype=g.dtype, device=g.device)
        _check(lib().mm_moe_unpermute(g.contiguous().data_ptr(), row_of_pair.data_ptr(), ones.data_ptr(), out.data_ptr(),
                                      ctx.T, ctx.k, g.shape[1], _st()), "moe_unpermute")
        return out, None, None, None


class _AlignedUnpermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, row_of_pair, probs):
        T, k = probs.shape
        out = torch.empty(T, y.shape[1], dtype=y.dtype, device=y.device)
        pc = probs.to(y.dtype).contiguous()
        _check(lib().mm_moe_unpermute(y.contiguous().data_ptr(), row_of_pair.data_ptr(), pc.data_ptr(), out.data_ptr(), T, k,
                                      y.shape[1], _st()), "moe_unpermute")
        ctx.save_for_backward(y, row_of_pair, pc)
        return out

    @staticmethod
    def backward(ctx, g):
        y, row_of_pair, probs = ctx.saved_tensors
        T, k = probs.shape
        idx = row_of_pair.long()
        ge = g.repeat_interleave(k, dim=0)                              # [T*k, H]
        dy = torch.zeros_like(y)
        dy[idx] = ge * probs.reshape(-1, 1)
        dprobs = (ge.float() * y[idx].float()).sum(-1).view(T, k).to(probs.dtype)
        return dy, None, dprobs


def _grouped_raw(a, b, c, off, mode, K, N, E):
    R = a.shape[0]
    plan = torch.empty(3 * lib().mm_grouped_gemm_max_tiles(R, E, K, N, mode) + 1, dtype=torch.int32, device=a.device)
    _check(lib().mm_grouped_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), off.data_ptr(), plan.data_ptr(), R, E, K, N,
                                      mode, status_word(a.device).data_ptr(), _st()), "grouped_gemm")


class _AlignedGroupedGemm(torch.autograd.Function):
    """x [R, K] (aligned expert-major rows) x W [E, K, N] -> [R, N]; all three passes on tcgen05."""

    @staticmethod
    def forward(ctx, x, w, off):
        E, K, N = w.shape
        x = x.contiguous()
        y = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        _grouped_raw(x, w, y, off, 0, K, N, E)
        ctx.save_for_backward(x, w, off)
        return y

    @staticmethod
    def backward(ctx, g):
        x, w, off = ctx.saved_tensors
        E, K, N = w.shape
        g = g.contiguous()
        dx = torch.empty_like(x)
        _grouped_raw(g, w, dx, off, 1, K, N, E)
        dw = torch.zeros_like(w)
        _grouped_raw(x, g, dw, off, 2, K, N, E)
        return dx, dw, None


def moe_experts(tokens, topk_ids, probs, gate_up, down):
    """Routed SwiGLU experts: permute -> grouped GEMM -> SwiGLU -> grouped GEMM -> weighted un-permute."""
    E = gate_up.shape[0]
    off, row_of_pair, src_of_row, R = aligned_routing(topk_ids, E)
    x = _AlignedPermute.apply(tokens, src_of_row, row_of_pair, topk_ids.shape[1])
    h = _AlignedGroupedGemm.apply(x, gate_up, off)
    y = _AlignedGroupedGemm.apply(swiglu(h), down, off)
    return _AlignedUnpermute.apply(y, row_of_pair, probs)


# --------------------------------------------------------------------------- GDN
def _seq_bounds(cu_seqlens, T, device):
    """Per-token first index and one-past-last index of its sequence (int32 [T] each)."""
    if cu_seqlens is None:
        return (torch.zeros(T, dtype=torch.int32, device=device), torch.full((T,), T, dtype=torch.int32, device=device))
    cu = torch.as_tensor(cu_seqlens, device=device).to(torch.int64)
    seg = torch.bucketize(torch.arange(T, device=device), cu[1:], right=True)
    return cu[seg].int().contiguous(), cu[seg + 1].int().contiguous()


class _CausalConv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cu_seqlens, silu):
        T, D = x.shape
        K = w.shape[-1]
        x, w = x.contiguous(), w.contiguous()
        start, end = _seq_bounds(cu_seqlens, T, x.device)
        y = torch.empty_like(x)
        _check(lib().mm_conv1d_fwd(x.data_ptr(), w.data_ptr(), start.data_ptr(), y.data_ptr(), T, D, K, int(silu), _st()),
               "conv1d_fwd")
        ctx.save_for_backward(x, w, start, end)
        ctx.silu = silu
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, start, end = ctx.saved_tensors
        T, D = x.shape
        K = w.shape[-1]
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros(D, K, dtype=torch.float32, device=x.device)
        _check(lib().mm_conv1d_bwd(x.data_ptr(), w.data_ptr(), start.data_ptr(), end.data_ptr(), dy.data_ptr(),
                                   dx.data_ptr(), dw.data_ptr(), T, D, K, int(ctx.silu), _st()), "conv1d_bwd")
        return dx, dw.to(w.dtype), None, None


def conv1d_supported(x, w) -> bool:
    return x.dim() == 2 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 \
        and w.shape[-1] <= 8


def causal_conv1d(x, w, activation, cu_seqlens):
    return _CausalConv1d.apply(x, w, cu_seqlens, activation == "silu")


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D).contiguous()
        y = torch.empty_like(x2)
        r = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        fn = lib().mm_l2norm_fwd if (D % 8 or not _row_group(D)) else lib().mm_rownorm_l2_fwd
        _check(fn(x2.data_ptr(), y.data_ptr(), r.data_ptr(), x2.shape[0], D, eps, _st()), "l2norm_fwd")
        ctx.save_for_backward(y, r)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        y, r = ctx.saved_tensors
        D = y.shape[-1]
        dy2 = dy.reshape(-1, D).contiguous()
        dx = torch.empty_like(y)
        _check(lib().mm_l2norm_bwd(y.data_ptr(), dy2.data_ptr(), r.data_ptr(), dx.data_ptr(), y.shape[0], D, _st()),
               "l2norm_bwd")
        return dx.view(dy.shape), None


def l2_norm(x, eps=1e-6):
    return _L2Norm.apply(x, eps)


class _GatedRMSNorm(torch.autograd.Function):
    """``rmsnorm(x) * w * silu(z)`` over the last dim (<= 256): x fp32 or bf16, z / w / result bf16."""

    @staticmethod
    def forward(ctx, x, z, w, eps):
        D = x.shape[-1]
        x2, z2, wc = x.reshape(-1, D).contiguous(), z.reshape(-1, D).contiguous(), w.contiguous()
        rows = x2.shape[0]
        y = torch.empty(rows, D, dtype=torch.bfloat16, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(lib().mm_gated_rms_fwd(x2.data_ptr(), int(x2.dtype == torch.float32), z2.data_ptr(), wc.data_ptr(), y.data_ptr(),
                                      rstd.data_ptr(), rows, D, eps, _st()), "gated_rms_fwd")
        ctx.save_for_backward(x2, z2, wc, rstd)
        ctx.shapes = (x.shape, z.shape)
        return y.view(z.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, z2, wc, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = dy.reshape(rows, D).contiguous()
        dx, dz = torch.empty_like(x2), torch.empty_like(z2)
        dw = torch.zeros(D, dtype=torch.float32, device=x2.device)
        _check(lib().mm_gated_rms_bwd(x2.data_ptr(), int(x2.dtype == torch.float32), z2.data_ptr(), wc.data_ptr(), dy2.data_ptr(),
                                      rstd.data_ptr(), dx.data_ptr(), dz.data_ptr(), dw.data_ptr(), rows, D, _st()),
               "gated_rms_bwd")
        return dx.view(ctx.shapes[0]), dz.view(ctx.shapes[1]), dw.to(wc.dtype), None


def gated_rms_norm(x, z, w, eps=1e-6):
    return _GatedRMSNorm.apply(x, z, w, eps)


def gdn_supported(q, v, chunk) -> bool:
    from . import gdn
    lib()
    return _STATUS.get("mm_gdn_fwd", False) and gdn.supported(q, v, chunk)


def gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, chunk, scale):
    from . import gdn
    return gdn.gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, scale)
