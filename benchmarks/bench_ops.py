"""Per-kernel timing on one GPU: CUDA events, >=3 warm-ups, L2 flushed between timed iterations.

    python benchmarks/bench_ops.py [--ops gemm,gemm_swiglu,elementwise,lce,fmha,gdn,vit_attention,grouped_gemm,small_ops,sparse_attention] [--out FILE] [--small]

Prints one JSON line per case: achieved TFLOP/s or GB/s and the fraction of the measured peaks in
MEASURED_PEAKS.json (fallback 1590 TFLOP/s / 6650 GB/s when the file is absent).  ``--small`` keeps
inputs just above L2 size so that a profiler capture of the same command stays short.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.ops import native  # noqa: E402
from mindspeed_mm_b200.ops import reference as ref  # noqa: E402


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


_flush = None


def time_fn(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def emit(rec, out):
    line = json.dumps(rec)
    print(line, flush=True)
    if out:
        with open(out, "a") as f:
            f.write(line + "\n")


def bench_gemm(out, small):
    tf, _, src = peaks()
    shapes = [("qkv", 8192, 4608, 3584), ("o", 8192, 3584, 3584), ("gate_up", 8192, 37888, 3584),
              ("down", 8192, 3584, 18944), ("square", 8192, 8192, 8192), ("vit_qkv", 8192, 3840, 1280)]
    if small:
        shapes = [("qkv", 8192, 4608, 3584)]
    for name, M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        bt = b.t().contiguous()
        at = a.t().contiguous()
        flops = 2.0 * M * N * K
        cases = [("nt", lambda: native.gemm_nt(a, b), lambda: a @ b.t()),
                 ("nn", lambda: native.gemm_nn(a, bt), lambda: a @ bt),
                 ("tn", lambda: native.gemm_tn(at, bt), lambda: at.t() @ bt)]
        for lay, mine, lib in cases:
            t = time_fn(mine)
            tl = time_fn(lib)
            emit(dict(op="gemm_bf16", case=name, layout=lay, M=M, N=N, K=K, ms=round(t, 4),
                      tflops=round(flops / t / 1e9, 1), frac_of_peak=round(flops / t / 1e9 / tf, 3), peak=src,
                      cublas_ms=round(tl, 4), cublas_tflops=round(flops / tl / 1e9, 1),
                      vs_cublas=round(tl / t, 3)), out)
        native.check_status()


def bench_gemm_swiglu(out, small):
    """gate/up projection + SwiGLU: one kernel with the activation as the epilogue against GEMM followed by the activation
    kernel (the decoder MLP of Qwen2.5-VL-7B, and the ViT-sized one)."""
    tf, _, src = peaks()
    shapes = [("llm_mlp", 8192, 18944, 3584)] if small else [("llm_mlp", 8192, 18944, 3584), ("mlp_5120", 8192, 13824, 5120)]
    for name, M, F, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(2 * F, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
        flops = 4.0 * M * F * K
        with torch.no_grad():
            t_f = time_fn(lambda: native.gemm_swiglu(x, w))
            t_u = time_fn(lambda: native.swiglu(native.gemm_nt(x, w)))
            t_l = time_fn(lambda: native.swiglu(x @ w.t()))
        emit(dict(op="gemm_swiglu_bf16", case=name, M=M, F=F, K=K, fused_ms=round(t_f, 4),
                  fused_tflops=round(flops / t_f / 1e9, 1), frac_of_peak=round(flops / t_f / 1e9 / tf, 3), peak=src,
                  gemm_then_act_ms=round(t_u, 4), cublas_then_act_ms=round(t_l, 4), vs_two_kernels=round(t_u / t_f, 3)), out)
        native.check_status()


ONLY: list = []      # --only a,b: restrict a benchmark to the rows whose name contains one of the words (for short profiler captures)


def want(name: str) -> bool:
    return not ONLY or any(o in name for o in ONLY)


def bench_elementwise(out, small):
    _, bw, src = peaks()
    T = 8192 if small else 32768
    H = 3584
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(x)

    def rec(name, fn, nbytes, base=None, width=H):
        if not want(name):
            return
        t = time_fn(fn)
        r = dict(op=name, T=T, H=width, ms=round(t, 4), gbs=round(nbytes / t / 1e6, 1),
                 frac_of_peak=round(nbytes / t / 1e6 / bw, 3), peak=src)
        if base is not None:
            tb = time_fn(base)
            r.update(torch_ms=round(tb, 4), vs_torch=round(tb / t, 2))
        emit(r, out)

    ops.set_tier("native")
    rec("rmsnorm_fwd", lambda: ops.rms_norm(x, w, 1e-6), 2 * x.numel() * 2,
        lambda: torch.nn.functional.rms_norm(x, (H,), w, 1e-6))
    native.lib().mm_rmsnorm_set_v16(0)          # the 16-byte-access form of the same kernel, for comparison
    rec("rmsnorm_fwd_16B_accesses", lambda: ops.rms_norm(x, w, 1e-6), 2 * x.numel() * 2)
    native.lib().mm_rmsnorm_set_v16(1)
    xg = x.clone().requires_grad_()
    wg = w.clone().requires_grad_()
    y = ops.rms_norm(xg, wg, 1e-6)
    rec("rmsnorm_bwd", lambda: torch.autograd.grad(y, (xg, wg), dy, retain_graph=True), 3 * x.numel() * 2)
    F = 18944
    gu = torch.randn(T // 4, 2 * F, device="cuda", dtype=torch.bfloat16)
    rec("swiglu_fwd", lambda: ops.swiglu(gu), gu.numel() * 2 * 1.5,
        lambda: torch.nn.functional.silu(gu[:, :F]) * gu[:, F:])
    if want("adamw_shard"):
        n = 256 << 20 if not small else 32 << 20
        p, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
        g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
        p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        rec("adamw_shard", lambda: native.adamw_shard(p, m, v, g, p16, 1e-4, 0.9, 0.999, 1e-8, 0.0, 1, n, 1.0), n * 28.0)
        del p, m, v, g, p16
    # DiT-side ops: adaLN modulate and gated residual on [B, S, H] with per-sample [B, 1, H] vectors; rotary on [T, N, D]
    Hd = 5120
    xd = torch.randn(1, T, Hd, device="cuda", dtype=torch.bfloat16)
    sc, sh, gt = (torch.randn(1, 1, Hd, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    yd = torch.randn_like(xd)
    rec("layer_norm_modulate", lambda: ops.layer_norm_modulate(xd, sc, sh, 1e-6), 2 * xd.numel() * 2,
        lambda: ref.layer_norm_modulate(xd, sc, sh, 1e-6), width=Hd)
    rec("gated_residual", lambda: ops.gated_residual(xd, yd, gt), 3 * xd.numel() * 2, lambda: ref.gated_residual(xd, yd, gt),
        width=Hd)
    q = torch.randn(T, 28, 128, device="cuda", dtype=torch.bfloat16)
    ang = torch.randn(T, 64, device="cuda")
    cos, sin = torch.cat([ang.cos()] * 2, -1).to(torch.bfloat16), torch.cat([ang.sin()] * 2, -1).to(torch.bfloat16)
    rec("rope_rotate_half", lambda: ops.rope_rotate_half(q, cos, sin), 2 * q.numel() * 2, lambda: ref.rope_rotate_half(q, cos, sin))


def bench_lce(out, small):
    """Fused final projection + cross entropy, forward and backward, against materialised logits."""
    tf, _, src = peaks()
    T, H, V = (4096, 3584, 32768) if small else (8192, 3584, 152064)
    h = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    ops.set_tier("native")

    def mine():
        loss, n = ops.linear_cross_entropy(h, w, labels)
        torch.autograd.grad(loss / n, (h, w))

    def plain():
        loss = torch.nn.functional.cross_entropy((h @ w.t()).float(), labels)
        torch.autograd.grad(loss, (h, w))

    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    t = time_fn(mine, iters=5)
    mem = (torch.cuda.max_memory_allocated() - base) / 2 ** 30
    torch.cuda.reset_peak_memory_stats()
    tb = time_fn(plain, iters=5)
    mem_b = (torch.cuda.max_memory_allocated() - base) / 2 ** 30
    flops = 3 * 2.0 * T * H * V
    emit(dict(op="linear_cross_entropy_fwd_bwd", T=T, H=H, V=V, ms=round(t, 3), tflops=round(flops / t / 1e9, 1),
              frac_of_peak=round(flops / t / 1e9 / tf, 3), peak=src, extra_mem_gb=round(mem, 2), torch_ms=round(tb, 3),
              torch_extra_mem_gb=round(mem_b, 2), vs_torch=round(tb / t, 2)), out)
    native.check_status()


def bench_fmha(out_file, small):
    import math
    tf, _, src = peaks()
    from flash_attn import flash_attn_varlen_func
    cases = [("llm_causal_4x2048", [2048] * 4, 28, 4, True), ("dit_full_1x16384", [16384], 8, 8, False)]
    if not small:
        cases.append(("dit_full_1x75600_5heads", [75600], 5, 5, False))
    for name, lens, nq, nkv, causal in cases:
        T, D = sum(lens), 128
        q = torch.randn(T, nq, D, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(T, nkv, D, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(T, nkv, D, device="cuda", dtype=torch.bfloat16)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        flops = sum(4.0 * l * l * D * nq for l in lens) * (0.5 if causal else 1.0)
        sc = 1.0 / math.sqrt(D)
        t = time_fn(lambda: native.fmha_forward(q, k, v, cu, cu, causal, sc))
        tl = time_fn(lambda: flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=causal))
        # backward: tcgen05 dQ + dK/dV kernels against flash-attn's backward, both fed with the native forward's out / lse
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward
        out, lse = native.fmha_forward(q, k, v, cu, cu, causal, sc)
        do = torch.randn_like(out)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        tb = time_fn(lambda: native.fmha_backward(do, q, k, v, out, lse, cu, cu, causal, sc), iters=5)
        tbl = time_fn(lambda: _flash_attn_varlen_backward(do, q, k, v, out, lse, dq, dk, dv, cu, cu, max(lens), max(lens), 0.0,
                                                          sc, causal, -1, -1, 0.0, None, False), iters=5)
        emit(dict(op="fmha_bwd", case=name, T=T, heads=nq, kv_heads=nkv, causal=causal, ms=round(tb, 4),
                  tflops=round(2.5 * flops / tb / 1e9, 1), frac_of_peak=round(2.5 * flops / tb / 1e9 / tf, 3), peak=src,
                  flash_attn2_ms=round(tbl, 4), flash_attn2_tflops=round(2.5 * flops / tbl / 1e9, 1),
                  vs_flash_attn2=round(tbl / tb, 3)), out_file)
        emit(dict(op="fmha_fwd", case=name, T=T, heads=nq, kv_heads=nkv, causal=causal, ms=round(t, 4),
                  tflops=round(flops / t / 1e9, 1), frac_of_peak=round(flops / t / 1e9 / tf, 3), peak=src,
                  flash_attn2_ms=round(tl, 4), flash_attn2_tflops=round(flops / tl / 1e9, 1), vs_flash_attn2=round(tl / t, 3)), out_file)
        native.check_status()


def bench_vit_attention(out_file, small):
    """Vision-tower attention of Qwen2.5-VL: 8 images of 448 x 448 = 8192 patches, 16 heads of 80; the window layers
    (128 windows of 64 tokens) and the full-attention layers (8 sequences of 1024), forward and backward, against
    flash-attn 2 on the same tensors."""
    import math
    from flash_attn import flash_attn_varlen_func
    tf, hbm, src = peaks()
    T, N, D = 8192, 16, 80
    for name, lens in (("vit_windows_128x64", [64] * 128), ("vit_full_8x1024", [1024] * 8)):
        qkv = torch.randn(T, 3, N, D, device="cuda", dtype=torch.bfloat16)
        q, k, v = qkv.unbind(1)                                  # strided views of the fused projection, as in the model
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        sc = 1.0 / math.sqrt(D)
        flops = sum(4.0 * l * l * D * N for l in lens)
        bytes_ = 4.0 * T * N * D * 2
        t = time_fn(lambda: native.fmha_forward(q, k, v, cu, cu, False, sc))
        tl = time_fn(lambda: flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=False))
        out, lse = native.fmha_forward(q, k, v, cu, cu, False, sc)
        do = torch.randn_like(out)
        tb = time_fn(lambda: native.fmha_backward(do, q, k, v, out, lse, cu, cu, False, sc), iters=5)
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward
        qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
        dq, dk, dv = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
        tbl = time_fn(lambda: _flash_attn_varlen_backward(do, qc, kc, vc, out, lse, dq, dk, dv, cu, cu, max(lens), max(lens), 0.0,
                                                          sc, False, -1, -1, 0.0, None, False), iters=5)
        emit(dict(op="vit_attention", case=name, T=T, heads=N, head_dim=D, fwd_ms=round(t, 4), bwd_ms=round(tb, 4),
                  fwd_tflops=round(flops / t / 1e9, 1), fwd_gbs=round(bytes_ / t / 1e6, 1),
                  fwd_frac_of_hbm=round(bytes_ / t / 1e6 / hbm, 3), peak=src, flash_attn2_fwd_ms=round(tl, 4),
                  flash_attn2_bwd_ms=round(tbl, 4), fwd_vs_flash_attn2=round(tl / t, 3), bwd_vs_flash_attn2=round(tbl / tb, 3)),
             out_file)
        native.check_status()


def bench_grouped_gemm(out, small):
    """Grouped expert GEMMs of Qwen3-VL-30B-A3B on one EP rank of 8: 16 local experts, 8192 tokens x top-8 / 8 ranks =
    8192 routed rows with a skewed histogram (softmax of N(0, 0.8) logits); gate_up [2048 -> 1536] and down [768 -> 2048].
    The native kernel works on the aligned expert-major layout (every expert's rows start at a multiple of 128); it is
    timed forward and forward + data gradient + weight gradient against a loop of cuBLAS matmuls over the experts' true
    row ranges of the same buffer."""
    tf, _, src = peaks()
    E, H, F = 16, 2048, 768
    rows = 8192 if not small else 2048
    g = torch.Generator().manual_seed(0)
    w = torch.softmax(torch.randn(E, generator=g) * 0.8, 0)
    ids = torch.multinomial(w, rows, replacement=True, generator=g).view(rows, 1).cuda()
    counts = torch.bincount(ids.view(-1), minlength=E).tolist()
    off, _, _, R = native.aligned_routing(ids, E)
    starts = off.tolist()
    for name, K, N in (("gate_up", H, 2 * F), ("down", F, H)):
        x = torch.randn(R, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        wt = (torch.randn(E, K, N, device="cuda") / K ** 0.5).to(torch.bfloat16).requires_grad_()
        flops = 2.0 * rows * K * N

        def fwd_native():
            return native._AlignedGroupedGemm.apply(x, wt, off)

        class Loop(torch.autograd.Function):
            @staticmethod
            def forward(ctx, x, wt):
                ctx.save_for_backward(x, wt)
                y = torch.empty(R, N, dtype=x.dtype, device=x.device)
                for e in range(E):
                    if counts[e]:
                        torch.matmul(x[starts[e]:starts[e] + counts[e]], wt[e], out=y[starts[e]:starts[e] + counts[e]])
                return y

            @staticmethod
            def backward(ctx, gy):
                x, wt = ctx.saved_tensors
                dx, dw = torch.empty_like(x), torch.zeros_like(wt)
                for e in range(E):
                    if counts[e]:
                        sl = slice(starts[e], starts[e] + counts[e])
                        torch.matmul(gy[sl], wt[e].t(), out=dx[sl])
                        torch.matmul(x[sl].t(), gy[sl], out=dw[e])
                return dx, dw

        def fwd_loop():
            return Loop.apply(x, wt)
        t_f = time_fn(lambda: fwd_native())
        t_fl = time_fn(lambda: fwd_loop())
        gy = torch.randn(R, N, device="cuda", dtype=torch.bfloat16)

        def bwd(fn):
            x.grad = wt.grad = None
            fn().backward(gy)
        t_fb = time_fn(lambda: bwd(fwd_native), iters=5)
        t_fbl = time_fn(lambda: bwd(fwd_loop), iters=5)
        emit(dict(op="grouped_gemm", case=name, rows=rows, aligned_rows=int(starts[-1]), experts=E, K=K, N=N,
                  max_rows=max(counts), min_rows=min(counts),
                  fwd_ms=round(t_f, 4), fwd_tflops=round(flops / t_f / 1e9, 1), fwd_frac_of_peak=round(flops / t_f / 1e9 / tf, 3),
                  fwd_bwd_ms=round(t_fb, 4), fwd_bwd_tflops=round(3 * flops / t_fb / 1e9, 1),
                  fwd_bwd_frac_of_peak=round(3 * flops / t_fb / 1e9 / tf, 3), peak=src,
                  cublas_loop_fwd_ms=round(t_fl, 4), cublas_loop_fwd_bwd_ms=round(t_fbl, 4),
                  fwd_vs_cublas_loop=round(t_fl / t_f, 3), fwd_bwd_vs_cublas_loop=round(t_fbl / t_fb, 3)), out)
        native.check_status()


def bench_small_ops(out, small):
    """Memory-bound kernels without an earlier measurement: depthwise causal conv1d (+SiLU), L2 norm, GELU, affine
    LayerNorm.  Bytes = one read + one write of the activation (plus the gradient traffic for backward)."""
    import torch.nn.functional as F
    _, hbm, src = peaks()
    T = 65536 if not small else 16384

    def rec(name, fn, nbytes, eager=None, **kw):
        t = time_fn(fn)
        r = dict(op=name, ms=round(t, 4), gbs=round(nbytes / t / 1e6, 1), frac_of_hbm=round(nbytes / t / 1e6 / hbm, 3), peak=src, **kw)
        if eager is not None:
            te = time_fn(eager)
            r.update(eager_ms=round(te, 4), vs_eager=round(te / t, 3))
        emit(r, out)
    x = torch.randn(T, 4096, device="cuda", dtype=torch.bfloat16)
    nb = 2.0 * x.numel() * 2
    rec("gelu_tanh_fwd", lambda: ops.gelu_tanh(x), nb, lambda: F.gelu(x, approximate="tanh"), T=T, H=4096)
    w = torch.ones(4096, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(4096, device="cuda", dtype=torch.bfloat16)
    rec("layer_norm_affine_fwd", lambda: ops.layer_norm(x, w, b), nb, lambda: F.layer_norm(x, (4096,), w, b), T=T, H=4096)
    xn = torch.randn(T, 32, 128, device="cuda", dtype=torch.bfloat16)
    rec("l2_norm_fwd", lambda: ops.l2_norm(xn), 2.0 * xn.numel() * 2, lambda: F.normalize(xn.float(), dim=-1).to(xn.dtype),
        T=T, heads=32, D=128)
    xc = torch.randn(T, 8192, device="cuda", dtype=torch.bfloat16)
    wc = torch.randn(8192, 4, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, T // 2, T], dtype=torch.int32, device="cuda")
    rec("causal_conv1d_silu_fwd", lambda: ops.causal_conv1d(xc, wc, None, "silu", cu), 2.0 * xc.numel() * 2,
        lambda: ref.causal_conv1d(xc, wc, None, "silu", cu), T=T, channels=8192, width=4)
    native.check_status()


def bench_gdn(out, small):
    """Gated delta rule, K = V = 128, chunk 64: the state-pass kernel alone, the whole operator (batched prologue
    + kernel), forward + backward, and the PyTorch chunked oracle on the same GPU."""
    from mindspeed_mm_b200.ops import gdn, reference as ref
    import torch.nn.functional as F
    cases = [("4x2048_h16", [2048] * 4, 16)] + ([] if small else [("2x8192_h32", [8192] * 2, 32)])
    for name, lens, H in cases:
        T = sum(lens)
        cu = [0] + [int(c) for c in torch.tensor(lens).cumsum(0)]
        q = F.normalize(torch.randn(T, H, 128, device="cuda"), dim=-1).bfloat16()
        k = F.normalize(torch.randn(T, H, 128, device="cuda"), dim=-1).bfloat16()
        v = torch.randn(T, H, 128, device="cuda", dtype=torch.bfloat16)
        g = -0.5 * torch.rand(T, H, device="cuda")
        beta = torch.rand(T, H, device="cuda")
        lay = gdn._layout(cu, q.device)
        with torch.no_grad():
            pro = gdn.chunk_prologue(*(lay.scatter(t.float()) for t in (q, k, v, g, beta)), 128 ** -0.5)
            args = [t.to(torch.bfloat16).contiguous() for t in pro[:5]] + [pro[5].float().contiguous()]
            t_kernel = time_fn(lambda: gdn._state_pass_native(*args, lay, False))
            t_fwd = time_fn(lambda: gdn.gated_delta_rule_varlen(q, k, v, g, beta, cu))
            t_ref = time_fn(lambda: [ref.gated_delta_rule_chunked(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b],
                                                                  beta[None, a:b]) for a, b in zip(cu[:-1], cu[1:])],
                            iters=3, warmup=1)
        ins = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]

        def fb():
            o = gdn.gated_delta_rule_varlen(*ins, cu)
            o.backward(torch.ones_like(o))
        t_fb = time_fn(fb, iters=5)
        NC = lay.NC
        # tensor-core work of the state pass per chunk and head: D1, D2 (2 x 2*128*64*128), O (2*128*64*64), S (2*128*64*128)
        flops = NC * H * (3 * 2 * 128 * 64 * 128 + 2 * 128 * 64 * 64)
        bytes_ = NC * H * 64 * (3 * 128 + 64 + 2 * 128) * 2          # W, Qg, Kd, At, U in; O out
        emit(dict(op="gdn", case=name, T=T, heads=H, chunks=NC, state_pass_ms=round(t_kernel, 4),
                  state_pass_tflops=round(flops / t_kernel / 1e9, 1), state_pass_gbs=round(bytes_ / t_kernel / 1e6, 1),
                  fwd_ms=round(t_fwd, 3), fwd_bwd_ms=round(t_fb, 3), torch_chunked_fwd_ms=round(t_ref, 3),
                  fwd_vs_torch_chunked=round(t_ref / t_fwd, 2)), out)
        native.check_status()


def bench_sparse_attention(out, small):
    """Sliding-tile attention of a video DiT (HunyuanVideo-1.5 layout: tiles of 6 x 8 x 8 = 384 tokens, 3 x 3 x 3 window,
    256 trailing text tokens) against dense attention over the same tokens, forward and forward + backward; the sparse
    path is the gather of the selected key blocks + one packed varlen call."""
    from mindspeed_mm_b200.ops import sparse_attention as sa
    cases = [("12x32x48", (12, 32, 48), 8)] if small else [("18x48x80", (18, 48, 80), 8), ("30x48x80", (30, 48, 80), 8)]
    for name, canvas, N in cases:
        S = canvas[0] * canvas[1] * canvas[2] + 256
        q, k, v = (torch.randn(1, S, N, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        with torch.no_grad():
            _, density = sa.ssta_attention(q, k, v, canvas, kernel=(3, 3, 3), text_len=256, mode="sta")
            t_sta = time_fn(lambda: sa.ssta_attention(q, k, v, canvas, kernel=(3, 3, 3), text_len=256, mode="sta"), iters=5)
            t_dense = time_fn(lambda: ops.attention_dense(q, k, v), iters=5)
        ins = [t.clone().requires_grad_() for t in (q, k, v)]

        def fb(mode):
            o = sa.ssta_attention(*ins, canvas, kernel=(3, 3, 3), text_len=256, mode=mode)[0]
            o.backward(torch.ones_like(o))
        t_sta_fb = time_fn(lambda: fb("sta"), iters=3, warmup=2)
        t_dense_fb = time_fn(lambda: fb("dense"), iters=3, warmup=2)
        emit(dict(op="sta_attention", case=name, tokens=S, heads=N, density=round(density, 3), sta_fwd_ms=round(t_sta, 3),
                  dense_fwd_ms=round(t_dense, 3), fwd_speedup=round(t_dense / t_sta, 2), sta_fwd_bwd_ms=round(t_sta_fb, 3),
                  dense_fwd_bwd_ms=round(t_dense_fb, 3), fwd_bwd_speedup=round(t_dense_fb / t_sta_fb, 2)), out)
        native.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="gemm,elementwise")
    ap.add_argument("--out", default="")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--only", default="", help="comma list of words: only the rows whose op name contains one of them")
    a = ap.parse_args()
    ONLY[:] = [w for w in a.only.split(",") if w]
    for op in a.ops.split(","):
        {"gemm": bench_gemm, "gemm_swiglu": bench_gemm_swiglu, "elementwise": bench_elementwise, "lce": bench_lce, "fmha": bench_fmha, "gdn": bench_gdn,
         "vit_attention": bench_vit_attention, "grouped_gemm": bench_grouped_gemm, "small_ops": bench_small_ops,
         "sparse_attention": bench_sparse_attention}[op](a.out, a.small)


if __name__ == "__main__":
    main()
