"""sm_100a kernels against plain fp32 PyTorch references of the same op."""
import math

import pytest
import torch

from mindspeed_mm_b200 import ops
from mindspeed_mm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, rtol=2e-2, atol=2e-2, rel_l2=1e-2, tile=128):
    """Three checks against the fp32 reference ``b``:
    * whole tensor: max |a - b| <= atol + rtol * max |b|
    * relative L2 error <= ``rel_l2`` (bf16 outputs of fp32-accumulated kernels sit near 3e-3), which a dropped K slice
      or a systematically wrong scale cannot meet
    * every ``tile`` x ``tile`` block of the 2-D view on its own: max error of the block <= rtol * max |b| of that
      block + 1e-3 * max |b| of the tensor, so a zeroed or stale tile of small values fails although it would hide
      under the whole-tensor maximum."""
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    scale = b.abs().max().item() + 1e-6
    assert err <= atol + rtol * scale, f"max err {err} vs scale {scale}"
    if rel_l2 is not None and b.numel() > 1:
        l2 = ((a - b).norm() / (b.norm() + 1e-12)).item()
        assert l2 <= rel_l2 or (a - b).abs().max().item() <= atol * 1e-2, f"relative L2 error {l2} > {rel_l2}"
    if tile and a.dim() >= 2 and a.shape[-1] >= tile:
        a2, b2 = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
        R, Cc = a2.shape
        pr, pc = (-R) % tile, (-Cc) % tile
        e2 = torch.nn.functional.pad((a2 - b2).abs(), (0, pc, 0, pr))
        s2 = torch.nn.functional.pad(b2.abs(), (0, pc, 0, pr))
        e_t = e2.view((R + pr) // tile, tile, (Cc + pc) // tile, tile).amax(dim=(1, 3))
        s_t = s2.view((R + pr) // tile, tile, (Cc + pc) // tile, tile).amax(dim=(1, 3))
        bad = e_t > rtol * s_t + 1e-3 * scale + 1e-6
        assert not bool(bad.any()), (f"{int(bad.sum())} of {bad.numel()} {tile}x{tile} tiles off; worst tile error "
                                     f"{float(e_t[bad].max())} against tile scale {float(s_t[bad][e_t[bad].argmax()])}")


@pytest.fixture(autouse=True)
def _native_tier():
    ops.set_tier("native")
    yield
    from mindspeed_mm_b200.ops import native
    native.check_status()


@pytest.mark.parametrize("T,H", [(333, 1280), (1024, 3584), (64, 8192), (7, 512), (4099, 128), (1000, 64), (300, 72),
                                 (130, 5120), (257, 1152), (3, 32)])
def test_rmsnorm_fwd_bwd(T, H):
    torch.manual_seed(0)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    y = ops.rms_norm(x, w, 1e-6)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rms_norm(xr, wr, 1e-6)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad, rtol=3e-2)


@pytest.mark.parametrize("T,F", [(257, 3424), (1024, 18944)])
def test_swiglu(T, F):
    torch.manual_seed(0)
    x = torch.randn(T, 2 * F, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(T, F, device=DEV, dtype=torch.bfloat16)
    y = ops.swiglu(x)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = ref.swiglu(xr)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)


@pytest.mark.parametrize("N,D", [(28, 128), (16, 80), (4, 128), (16, 72)])
def test_rope_half(N, D):
    torch.manual_seed(0)
    T = 515
    base = torch.randn(T, N * D + 64, device=DEV, dtype=torch.bfloat16)
    x = base[:, :N * D].view(T, N, D).detach().requires_grad_()          # strided view like q in fused qkv
    ang = torch.rand(T, D // 2, device=DEV) * 6.28
    emb = torch.cat([ang, ang], -1)
    cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)
    dy = torch.randn(T, N, D, device=DEV, dtype=torch.bfloat16)
    y = ops.rope_rotate_half(x, cos, sin)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = ref.rope_rotate_half(xr, cos.float(), sin.float())
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)


def test_rope_interleaved():
    torch.manual_seed(0)
    T, N, D = 300, 5, 128
    x = torch.randn(T, N, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    cos, sin = ref.rope3d_freqs((3, 10, 10), D, device=DEV)
    dy = torch.randn(T, N, D, device=DEV, dtype=torch.bfloat16)
    y = ops.rope_interleaved(x, cos, sin)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = ref.rope_interleaved(xr, cos, sin)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)


def test_ln_modulate_and_gated_residual():
    torch.manual_seed(0)
    B, S, H = 2, 301, 5120
    x = torch.randn(B, S, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    sc = (0.1 * torch.randn(B, 1, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    sh = (0.1 * torch.randn(B, 1, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(B, S, H, device=DEV, dtype=torch.bfloat16)
    y = ops.layer_norm_modulate(x, sc, sh, 1e-6)
    y.backward(dy)
    xr, scr, shr = (t.detach().float().requires_grad_() for t in (x, sc, sh))
    yr = ref.layer_norm_modulate(xr, scr, shr, 1e-6)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(sc.grad, scr.grad, rtol=3e-2)
    _close(sh.grad, shr.grad, rtol=3e-2)
    g = torch.randn(B, 1, H, device=DEV, dtype=torch.bfloat16)
    o = ops.gated_residual(x.detach(), y.detach(), g)
    _close(o, ref.gated_residual(x.detach().float(), y.detach().float(), g.float()))


def test_adamw_shard():
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    n = 128 * 1000
    p = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    for step in (1, 2, 3):
        g = torch.randn(n, device=DEV, dtype=torch.bfloat16)
        native.adamw_shard(p, m, v, g, p16, 1e-2, 0.9, 0.999, 1e-8, 0.1, step, n // 2, 0.5)
        ref.adamw_step(pr[:n // 2], mr[:n // 2], vr[:n // 2], g[:n // 2], 1e-2, 0.9, 0.999, 1e-8, 0.1, step, 0.5)
        ref.adamw_step(pr[n // 2:], mr[n // 2:], vr[n // 2:], g[n // 2:], 1e-2, 0.9, 0.999, 1e-8, 0.0, step, 0.5)
    _close(p, pr, rtol=1e-4, atol=1e-5)
    _close(m, mr, rtol=1e-4, atol=1e-6)
    _close(p16, pr, rtol=1e-2, atol=1e-2)


def test_rmsnorm_forward_access_widths_agree():
    """The 32-byte-access forward (rows that are a multiple of 16, 32-byte aligned) and the 16-byte form agree to a bf16
    rounding (their threads sum the squares in different groupings); a view at a 16-byte offset takes the 16-byte form."""
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    L = native.lib()
    for T, H in ((300, 3584), (64, 2048), (33, 8192), (17, 4080)):
        x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
        a = ops.rms_norm(x, w, 1e-6)
        L.mm_rmsnorm_set_v16(0)
        try:
            b = ops.rms_norm(x, w, 1e-6)
        finally:
            L.mm_rmsnorm_set_v16(1)
        assert (a.float() - b.float()).abs().max() <= 2 ** -6 * a.float().abs().max(), (T, H)
        _close(a, ref.rms_norm(x.float(), w.float(), 1e-6))
    buf = torch.randn(8 * 3584 + 8, device=DEV, dtype=torch.bfloat16)
    xo = buf[8:].view(8, 3584)                       # 16 bytes past a 32-byte boundary
    assert xo.data_ptr() % 32 == 16
    _close(ops.rms_norm(xo, w[:3584].contiguous(), 1e-6), ref.rms_norm(xo.float(), w[:3584].float(), 1e-6))


def test_sq_norm_of_shards():
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    shards = [torch.randn(n, device=DEV) * s for n, s in ((3, 1.0), (1021, 0.5), (128 * 1000, 2.0), (5_000_001, 0.1))]
    shards = [torch.cat([t.new_zeros(4), t])[4:] if t.numel() < 10 else t for t in shards]     # 16-byte aligned views
    got = native.sq_norm(shards)
    want = sum(float(t.double().pow(2).sum()) for t in shards)
    assert abs(float(got) - want) <= 1e-5 * want
    assert float(native.sq_norm(shards)) == float(got)          # fixed summation order


GEMM_SHAPES = [(128, 256, 64), (256, 512, 256), (1000, 768, 520), (8192, 4608, 3584), (333, 1280, 1176), (77, 136, 72),
               (1176, 1280, 8191 + 1), (3584, 152064 // 8, 512)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nt(M, N, K):
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    c = native.gemm_nt(a, b, bias)
    r = a.float() @ b.float().t() + bias.float()
    _close(c, r, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nn(M, N, K):
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    c = native.gemm_nn(a, b)
    _close(c, a.float() @ b.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K", [(m, n, k) for m, n, k in GEMM_SHAPES if m % 8 == 0])
def test_gemm_tn(M, N, K):
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    a = torch.randn(K, M, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    c = native.gemm_tn(a, b)
    _close(c, a.float().t() @ b.float(), rtol=1e-2, atol=1e-2)


def test_linear_autograd():
    torch.manual_seed(0)
    x = torch.randn(4, 130, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(768, 1024, device=DEV)).to(torch.bfloat16).requires_grad_()
    b = torch.randn(768, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(4, 130, 768, device=DEV, dtype=torch.bfloat16)
    y = ops.linear(x, w, b)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad)
    _close(b.grad, br.grad)


@pytest.mark.parametrize("T,H,V", [(300, 512, 32000), (1024, 1024, 152064)])
def test_linear_cross_entropy(T, H, V):
    torch.manual_seed(0)
    h = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (0.02 * torch.randn(V, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    lab = torch.randint(0, V, (T,), device=DEV)
    lab[::7] = -100
    loss, n = ops.linear_cross_entropy(h, w, lab)
    (loss / n).backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr, nr = ref.linear_cross_entropy(hr, wr, lab)
    (lr / nr).backward()
    assert abs(float(loss / n) - float(lr / nr)) < 2e-2 * float(lr / nr)
    _close(h.grad, hr.grad, rtol=5e-2, atol=1e-5)
    _close(w.grad, wr.grad, rtol=5e-2, atol=1e-5)


@pytest.mark.parametrize("lens,nq,nkv,causal", [([128], 1, 1, False), ([256, 128], 2, 1, False), ([300, 77, 513], 4, 2, True),
                                                  ([2048, 2048], 28, 4, True), ([1000], 5, 5, False)])
def test_fmha_forward_and_grad(lens, nq, nkv, causal):
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    T, D = sum(lens), 128
    qkv = torch.randn(T, (nq + 2 * nkv) * D, device=DEV, dtype=torch.bfloat16)
    q = qkv[:, :nq * D].view(T, nq, D)                       # strided views, like the model passes them
    k = qkv[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    out, lse = native.fmha_forward(q, k, v, cu, cu, causal, 1.0 / math.sqrt(D))
    ro, rl = ref.attention_varlen(q.float(), k.float(), v.float(), cu.cpu(), cu.cpu(), causal, return_lse=True)
    _close(out, ro, rtol=2e-2, atol=2e-2)
    assert (lse - rl).abs().max().item() < 2e-2
    # autograd path (native forward + backward fed with its out / lse)
    qg, kg, vg = (t.detach().clone().requires_grad_() for t in (q, k, v))
    o = ops.attention_varlen(qg, kg, vg, cu, cu, max(lens), max(lens), causal=causal)
    do = torch.randn_like(o)
    o.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = ref.attention_varlen(qr, kr, vr, cu.cpu(), cu.cpu(), causal)
    orf.backward(do.float())
    _close(qg.grad, qr.grad, rtol=3e-2, atol=3e-2)
    _close(kg.grad, kr.grad, rtol=3e-2, atol=3e-2)
    _close(vg.grad, vr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("fwd_variant,bwd_variant", [(0, 0), (3, 5)])
def test_fmha_kernel_variants_agree_with_reference(fwd_variant, bwd_variant):
    """The fallback forward / backward kernels stay correct beside the defaults: GQA + causal, ragged packing."""
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    lens, nq, nkv, D = [300, 129, 700], 4, 2, 128
    T = sum(lens)
    q, k, v = (torch.randn(T, n, D, device=DEV, dtype=torch.bfloat16) for n in (nq, nkv, nkv))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    prev_f = native.lib().mm_fmha_set_fwd_variant(fwd_variant)
    prev_b, native.FMHA_BWD_VARIANT = native.FMHA_BWD_VARIANT, bwd_variant
    try:
        qg, kg, vg = (t.detach().clone().requires_grad_() for t in (q, k, v))
        o = ops.attention_varlen(qg, kg, vg, cu, cu, max(lens), max(lens), causal=True)
        do = torch.randn_like(o)
        o.backward(do)
        native.check_status()
    finally:
        native.lib().mm_fmha_set_fwd_variant(prev_f)
        native.FMHA_BWD_VARIANT = prev_b
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = ref.attention_varlen(qr, kr, vr, cu.cpu(), cu.cpu(), True)
    orf.backward(do.float())
    _close(o, orf, rtol=2e-2, atol=2e-2)
    _close(qg.grad, qr.grad, rtol=3e-2, atol=3e-2)
    _close(kg.grad, kr.grad, rtol=3e-2, atol=3e-2)
    _close(vg.grad, vr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("D,lens,N,strided", [
    (80, [64] * 20 + [37, 256], 16, False),      # vision tower: 64-token windows, a ragged one, a full-image segment
    (80, [1024, 1024, 400], 16, True),           # vision tower full-attention layers, q/k/v views of a fused projection
    (64, [300, 129, 700], 4, False),
    (96, [130, 257], 2, False),
    # short sequences share 128-row tiles under a block-diagonal mask: ragged groups, a group of one, single tokens,
    # exact fits (64 + 64, 128), sequences longer than a tile in between
    (128, [30, 50, 48, 100, 20, 128, 200, 7, 1, 64, 64, 63, 2, 127, 1, 1], 4, False),
    (72, [16] * 9 + [100, 28, 5, 64], 2, True),
])
def test_attention_narrow_heads_run_the_tcgen05_kernels(D, lens, N, strided):
    """Head dims below 128 (a multiple of 8) run the same 128-wide kernels: the tensor maps carry the true head dim,
    TMA fills the missing columns with zeros and the stores skip them.  Nothing is padded in global memory and no
    library kernel runs (strict mode)."""
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    if strided:
        qkv = torch.randn(T, 3, N, D, device=DEV, dtype=torch.bfloat16)
        q, k, v = (t.detach().requires_grad_() for t in qkv.unbind(1))
    else:
        q, k, v = (torch.randn(T, N, D, device=DEV, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    before = native.LAUNCHES
    ops.set_strict(True)
    try:
        o = ops.attention_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=False)
        do = torch.randn_like(o)
        o.backward(do)
    finally:
        ops.set_strict(False)
    assert native.LAUNCHES > before and o.shape == (T, N, D)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = ref.attention_varlen(qr, kr, vr, cu.cpu(), cu.cpu(), False)
    orf.backward(do.float())
    _close(o, orf)
    _close(q.grad, qr.grad, rtol=3e-2, atol=3e-2)
    _close(k.grad, kr.grad, rtol=3e-2, atol=3e-2)
    _close(v.grad, vr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("tanh", [True, False])
def test_gelu_fwd_bwd(tanh):
    torch.manual_seed(0)
    x = (3 * torch.randn(333, 1280, device=DEV)).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(333, 1280, device=DEV, dtype=torch.bfloat16)
    y = ops.gelu_tanh(x) if tanh else ops.gelu(x)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = torch.nn.functional.gelu(xr, approximate="tanh" if tanh else "none")
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)


@pytest.mark.parametrize("shape,affine", [((2, 300, 1280), True), ((777, 5120), True), ((64, 1152), False)])
def test_layer_norm_affine_fwd_bwd(shape, affine):
    torch.manual_seed(0)
    H = shape[-1]
    x = torch.randn(*shape, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_() if affine else None
    b = (0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_() if affine else None
    dy = torch.randn(*shape, device=DEV, dtype=torch.bfloat16)
    ops.set_strict(True)
    try:
        y = ops.layer_norm(x, w, b, 1e-6)
        y.backward(dy)
    finally:
        ops.set_strict(False)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_() if affine else None
    br = b.detach().float().requires_grad_() if affine else None
    yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-6)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad, rtol=3e-2)
    if affine:
        _close(w.grad, wr.grad, rtol=3e-2, tile=0)
        _close(b.grad, br.grad, rtol=3e-2, tile=0)


def test_fallback_register_counts_and_strict_mode_refuses():
    """A call the kernels do not take (fp32 activations here) is counted by op name; strict mode raises instead."""
    x = torch.randn(8, 64, device=DEV)            # fp32: no kernel
    w = torch.ones(64, device=DEV)
    ops.library_fallbacks(reset=True)
    ops.rms_norm(x, w)
    assert ops.library_fallbacks(reset=True) == {"rms_norm": 1}
    ops.set_strict(True)
    try:
        with pytest.raises(RuntimeError):
            ops.rms_norm(x, w)
    finally:
        ops.set_strict(False)


def test_fmha_backward_cross_attention_shapes():
    """q and k/v of different lengths (DiT cross-attention to 512 text tokens), non-causal, tcgen05 backward."""
    torch.manual_seed(0)
    B, Sq, Sk, N, D = 2, 700, 512, 3, 128
    q = torch.randn(B, Sq, N, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, Sk, N, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, Sk, N, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    o = ops.attention_dense(q, k, v)
    do = torch.randn_like(o)
    o.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = ref.attention_dense(qr, kr, vr)
    orf.backward(do.float())
    _close(o, orf)
    _close(q.grad, qr.grad, rtol=3e-2, atol=3e-2)
    _close(k.grad, kr.grad, rtol=3e-2, atol=3e-2)
    _close(v.grad, vr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("M,K,F", [(300, 512, 256), (1024, 3584, 2048), (4100, 1024, 1152)])
def test_gemm_with_swiglu_epilogue_matches_reference(M, K, F):
    """Passes without a graph run the GEMM with the activation as its epilogue; a differentiated pass gives the same values."""
    from mindspeed_mm_b200.ops import native
    torch.manual_seed(0)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(2 * F, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    assert native.gemm_swiglu_supported(x, w)
    with torch.no_grad():
        fused = ops.linear_swiglu(x, w)
    gu = x.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    assert fused.shape == (M, F)
    _close(fused, want)
    xg = x.clone().requires_grad_()
    two_kernel = ops.linear_swiglu(xg, w)
    assert two_kernel.requires_grad
    _close(fused, two_kernel, rtol=1e-2, atol=1e-2)
    # 3-D input keeps its leading dims
    with torch.no_grad():
        assert ops.linear_swiglu(x.view(2, M // 2, K), w).shape == (2, M // 2, F)


def test_sliding_tile_attention_on_native_kernels_matches_masked_reference():
    """Block-sparse attention gathers the selected key blocks and runs the packed variable-length kernel; the oracle is a
    dense fp32 softmax under the token-level mask built from the same block mask."""
    from mindspeed_mm_b200.ops.sparse_attention import ssta_attention, sta_block_mask, tile_order
    torch.manual_seed(0)
    B, N, D = 1, 4, 128
    canvas, tile, kernel, text = (2, 8, 8), (1, 4, 4), (1, 3, 1), 16
    S = 2 * 8 * 8 + text
    q, k, v = (torch.randn(B, S, N, D, device=DEV, dtype=torch.bfloat16) * 0.5 for _ in range(3))
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    out, density = ssta_attention(q, k, v, canvas, tile, kernel=kernel, text_len=text, mode="sta")
    assert 0 < density < 1
    dy = torch.randn_like(out)
    out.backward(dy)
    # oracle
    block = 16
    tiles = (2, 2, 2)
    n_img = 8
    bm = torch.ones(n_img + 1, n_img + 1, dtype=torch.bool)
    bm[:n_img, :n_img] = sta_block_mask(tiles, kernel)
    perm = tile_order(canvas, tile)
    blk_of = torch.empty(S, dtype=torch.long)
    blk_of[perm] = torch.arange(n_img * block) // block
    blk_of[n_img * block:] = n_img
    tok_mask = bm[blk_of][:, blk_of].to(DEV)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    sc = torch.einsum("bqnd,bknd->bnqk", qr, kr) / math.sqrt(D)
    sc = sc.masked_fill(~tok_mask, float("-inf"))
    ref_out = torch.einsum("bnqk,bknd->bqnd", sc.softmax(-1), vr)
    ref_out.backward(dy.float())
    _close(out, ref_out)
    _close(q.grad, qr.grad)
    _close(k.grad, kr.grad)
    _close(v.grad, vr.grad)


@pytest.mark.parametrize("T,k,E,H,F", [(512, 2, 8, 256, 128), (4096, 8, 128, 2048, 768), (300, 4, 16, 512, 256)])
def test_moe_experts_native_vs_reference(T, k, E, H, F):
    torch.manual_seed(0)
    x = (torch.randn(T, H, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    gu = (torch.randn(E, H, 2 * F, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    dn = (torch.randn(E, F, H, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    logits = torch.randn(T, E, device=DEV)
    if E >= 16:
        logits[:, 0] += 2.0              # skewed routing: one hot expert, some experts may stay empty
        logits[:, E - 1] -= 30.0
    p, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    p = (p / p.sum(-1, keepdim=True)).to(torch.bfloat16).requires_grad_()
    y = ops.moe_experts(x, ids, p, gu, dn)
    g = torch.randn_like(y)
    y.backward(g)
    ops.set_tier("library")
    xr, gur, dnr, pr = (t.detach().float().requires_grad_() for t in (x, gu, dn, p))
    yr = ops.moe_experts(xr, ids, pr, gur, dnr)
    yr.backward(g.float())
    ops.set_tier("native")
    _close(y, yr, rtol=3e-2, atol=3e-2)
    _close(x.grad, xr.grad, rtol=4e-2, atol=4e-2)
    _close(gu.grad, gur.grad, rtol=4e-2, atol=4e-2)
    _close(dn.grad, dnr.grad, rtol=4e-2, atol=4e-2)
    _close(p.grad, pr.grad, rtol=4e-2, atol=4e-2)


@pytest.mark.parametrize("lens,D,K,silu", [([70, 200, 33], 512, 4, True), ([300], 1024, 4, False), ([5, 1, 64], 64, 3, True)])
def test_causal_conv1d_fwd_bwd(lens, D, K, silu):
    torch.manual_seed(0)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    x = torch.randn(T, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (0.5 * torch.randn(D, K, device=DEV)).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(T, D, device=DEV, dtype=torch.bfloat16)
    act = "silu" if silu else None
    y = ops.causal_conv1d(x, w, None, act, cu)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.causal_conv1d(xr, wr, None, act, cu.tolist())
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad, rtol=3e-2)


def test_l2norm_and_gated_rmsnorm():
    torch.manual_seed(0)
    x = torch.randn(777, 16, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn_like(x)
    y = ops.l2_norm(x)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = ref.l2_norm(xr)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    # gated RMSNorm, forward and backward, on the delta rule's fp32 output and on a bf16 input; a head dim that is
    # not a power-of-two number of vectors (72) as well
    for xdtype, D in ((torch.float32, 128), (torch.bfloat16, 128), (torch.float32, 72)):
        o = torch.randn(501, 8, D, device=DEV).to(xdtype).requires_grad_()
        z = torch.randn(501, 8, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
        gy = torch.randn(501, 8, D, device=DEV, dtype=torch.bfloat16)
        ops.set_strict(True)
        try:
            y = ops.gated_rms_norm(o, z, w, 1e-6)
            y.backward(gy)
        finally:
            ops.set_strict(False)
        orf, zr, wr = (t.detach().float().requires_grad_() for t in (o, z, w))
        yr = ref.gated_rms_norm(orf, zr, wr, 1e-6)
        yr.backward(gy.float())
        assert y.dtype == torch.bfloat16 and o.grad.dtype == xdtype
        _close(y, yr)
        _close(o.grad, orf.grad, rtol=3e-2, atol=3e-2)
        _close(z.grad, zr.grad, rtol=3e-2, atol=3e-2)
        _close(w.grad, wr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("lens,H", [([70, 200], 2), ([64], 1), ([1000, 130, 5], 4)])
def test_gated_delta_rule_native(lens, H):
    """tcgen05 state pass (+ hand-written backward) against the token-by-token fp32 recurrence."""
    torch.manual_seed(0)
    T, K, V = sum(lens), 128, 128
    cu = [0] + [int(c) for c in torch.tensor(lens).cumsum(0)]
    F = torch.nn.functional
    q = F.normalize(torch.randn(T, H, K, device=DEV), dim=-1).requires_grad_()
    k = F.normalize(torch.randn(T, H, K, device=DEV), dim=-1).requires_grad_()
    v = torch.randn(T, H, V, device=DEV).requires_grad_()
    g = (-0.5 * torch.rand(T, H, device=DEV)).requires_grad_()
    beta = torch.rand(T, H, device=DEV).requires_grad_()
    from mindspeed_mm_b200.ops import native
    assert native.gdn_supported(q, v, 64)
    o = ops.gated_delta_rule_varlen(q, k, v, g, beta, cu, chunk=64)
    do = torch.randn_like(o)
    grads = torch.autograd.grad(o, [q, k, v, g, beta], do)
    outs = []
    for a, b in zip(cu[:-1], cu[1:]):
        oo, _ = ref.gated_delta_rule_recurrent(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b], beta[None, a:b])
        outs.append(oo[0])
    o_ref = torch.cat(outs)
    grads_ref = torch.autograd.grad(o_ref, [q, k, v, g, beta], do)
    _close(o, o_ref, rtol=3e-2, atol=3e-3)
    for a, b in zip(grads, grads_ref):
        _close(a, b, rtol=5e-2, atol=5e-3)
    # a pass that keeps no graph runs the chunk-local prologue as one kernel on the packed tensors (bf16 in, as the layer
    # passes them): same result as the differentiated pass and as the recurrence
    with torch.no_grad():
        o_ng = ops.gated_delta_rule_varlen(q.bfloat16(), k.bfloat16(), v.bfloat16(), g, beta, cu, chunk=64)
    assert o_ng.dtype == torch.bfloat16
    _close(o_ng, o_ref, rtol=3e-2, atol=1e-2)
    _close(o_ng, o, rtol=3e-2, atol=1e-2)


@pytest.mark.parametrize("lens,H", [([70, 200], 2), ([1000, 130, 5], 3)])
def test_kimi_delta_attention_native(lens, H):
    """KDA on the tcgen05 state pass with one decay per key channel (+ hand-written backward) against the token-by-token
    fp32 recurrence."""
    torch.manual_seed(0)
    T, K, V = sum(lens), 128, 128
    cu = [0] + [int(c) for c in torch.tensor(lens).cumsum(0)]
    F = torch.nn.functional
    q = F.normalize(torch.randn(T, H, K, device=DEV), dim=-1).requires_grad_()
    k = F.normalize(torch.randn(T, H, K, device=DEV), dim=-1).requires_grad_()
    v = torch.randn(T, H, V, device=DEV).requires_grad_()
    g = (-0.1 * torch.rand(T, H, K, device=DEV)).requires_grad_()
    beta = torch.rand(T, H, device=DEV).requires_grad_()
    ops.library_fallbacks(reset=True)
    o = ops.kda_varlen(q, k, v, g, beta, cu)
    assert not ops.library_fallbacks(), ops.library_fallbacks()
    do = torch.randn_like(o)
    grads = torch.autograd.grad(o, [q, k, v, g, beta], do)
    outs = []
    for a, b in zip(cu[:-1], cu[1:]):
        oo, _ = ref.kda_recurrent(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b], beta[None, a:b])
        outs.append(oo[0])
    o_ref = torch.cat(outs)
    grads_ref = torch.autograd.grad(o_ref, [q, k, v, g, beta], do)
    _close(o, o_ref, rtol=3e-2, atol=3e-3)
    for a, b in zip(grads, grads_ref):
        _close(a, b, rtol=5e-2, atol=5e-3)
    # the batched [B, T, H, *] entry point takes the same path
    B, Tb = 2, 128
    sl = lambda t: t[: B * Tb].detach().reshape(B, Tb, *t.shape[1:])
    ob, _ = ops.kda(sl(q), sl(k), sl(v), sl(g), sl(beta))
    ob_ref, _ = ref.kda_recurrent(sl(q), sl(k), sl(v), sl(g), sl(beta))
    _close(ob, ob_ref, rtol=3e-2, atol=3e-3)


def test_expert_mlp_on_rows_grouped_by_expert_uses_the_aligned_kernels():
    """The all-to-all dispatcher hands over rows already grouped by expert (with empty experts): the aligned grouped
    kernels give the loop-of-matmuls result, forward and backward, and nothing falls back."""
    from mindspeed_mm_b200.parallel.ep import experts_mlp
    torch.manual_seed(0)
    E, H, Fi = 4, 256, 256
    counts = [130, 0, 77, 300]
    x = (torch.randn(sum(counts), H, device=DEV) * 0.5).bfloat16().requires_grad_()
    gu = (torch.randn(E, H, 2 * Fi, device=DEV) * 0.05).bfloat16().requires_grad_()
    dn = (torch.randn(E, Fi, H, device=DEV) * 0.05).bfloat16().requires_grad_()
    ops.library_fallbacks(reset=True)
    y = experts_mlp(x, gu, dn, counts)
    assert not ops.library_fallbacks(), ops.library_fallbacks()
    g = torch.randn_like(y)
    gx, ggu, gdn = torch.autograd.grad(y, [x, gu, dn], g)
    xr, gur, dnr = (t.detach().float().requires_grad_() for t in (x, gu, dn))
    outs, s0 = [], 0
    for e, c in enumerate(counts):
        h = xr[s0:s0 + c] @ gur[e]
        a, b = h.chunk(2, -1)
        outs.append((torch.nn.functional.silu(a) * b) @ dnr[e])
        s0 += c
    yr = torch.cat(outs)
    rx, rgu, rdn = torch.autograd.grad(yr, [xr, gur, dnr], g.float())
    _close(y, yr, rtol=3e-2, atol=3e-2)
    _close(gx, rx, rtol=3e-2, atol=3e-2)
    _close(ggu, rgu, rtol=3e-2, atol=5e-2)
    _close(gdn, rdn, rtol=3e-2, atol=5e-2)
    assert float(ggu[1].abs().max()) == 0.0 and float(gdn[1].abs().max()) == 0.0      # the empty expert


def test_peer_flag_wait_runs_out_and_reports_status():
    """Failure detection on the device without a fault: a wait on a flag that nothing sets gives up after its limit,
    the kernel returns, the status word says which kind of wait expired, and the context stays usable."""
    from mindspeed_mm_b200.ops import native
    L = native.lib()
    dev = torch.device(DEV)
    flags = torch.zeros(L.mm_p2p_flag_bytes() // 4, dtype=torch.int32, device=dev)
    assert L.mm_p2p_set_wait_limit(1 << 27) == 0                     # ~70 ms at 1.9 GHz
    try:
        native.status_word(dev).zero_()
        rc = L.mm_p2p_wait_done(flags.data_ptr(), 0, 1, 2, 0, native.status_word(dev).data_ptr(), native._st())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(native.status_word(dev).item()) == 4              # MM_TIMEOUT_PEER
        with pytest.raises(RuntimeError):
            native.check_status(dev)
    finally:
        assert L.mm_p2p_set_wait_limit(0) == 0
    x = torch.randn(64, 512, device=dev, dtype=torch.bfloat16)
    w = torch.ones(512, device=dev, dtype=torch.bfloat16)
    _close(ops.rms_norm(x, w), ref.rms_norm(x.float(), w.float()))
    assert int(native.status_word(dev).item()) == 0


def test_arena_barrier_wait_runs_out_then_passes():
    """The arena barrier is a kernel with a bounded wait: with a "peer" that never arrives (its flag lives in local
    memory and nothing writes it) the kernel gives up, reports MM_TIMEOUT_PEER and returns; once the flag is there the
    next barrier passes."""
    import ctypes as C
    from mindspeed_mm_b200.ops import native
    L = native.lib()
    dev = torch.device(DEV)
    n = L.mm_p2p_barrier_bytes() // 4
    blocks = torch.zeros(2, n, dtype=torch.int32, device=dev)        # rank 0's block (mine) and rank 1's
    ptrs = (C.c_void_p * 2)(blocks[0].data_ptr(), blocks[1].data_ptr())
    st = native.status_word(dev)
    assert L.mm_p2p_set_wait_limit(1 << 27) == 0
    try:
        st.zero_()
        assert L.mm_p2p_barrier(ptrs, 2, 0, 1, st.data_ptr(), native._st()) == 0
        torch.cuda.synchronize()
        assert int(st.item()) == 4
        assert blocks[0, 0].item() == 1 and blocks[1, 0].item() == 1     # my arrival was published to both blocks
        st.zero_()
        blocks[0, 1] = 2                                                  # the peer arrives at barrier 2
        assert L.mm_p2p_barrier(ptrs, 2, 0, 2, st.data_ptr(), native._st()) == 0
        torch.cuda.synchronize()
        assert int(st.item()) == 0
    finally:
        assert L.mm_p2p_set_wait_limit(0) == 0
        st.zero_()


def test_reduce_scatter_time_out_leaves_the_slot_usable():
    """A reduce-scatter launch whose peer never publishes its gradients skips the reduction, reports the time-out,
    and still completes its counter / done-flag protocol: the next launch on the same slot, with the peer present,
    reduces correctly."""
    import ctypes as C
    from mindspeed_mm_b200.ops import native
    L = native.lib()
    dev = torch.device(DEV)
    nflag = L.mm_p2p_flag_bytes() // 4
    flags = torch.zeros(2, nflag, dtype=torch.int32, device=dev)     # my flag block and the "peer's" (local memory)
    S = 1 << 14
    torch.manual_seed(0)
    g0 = torch.randn(2 * S, device=dev, dtype=torch.bfloat16)
    g1 = torch.randn(2 * S, device=dev, dtype=torch.bfloat16)
    gp = (C.c_void_p * 2)(g0.data_ptr(), g1.data_ptr())
    fp = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    out = torch.zeros(S, dtype=torch.float32, device=dev)
    st = native.status_word(dev)
    counter_idx, done_idx = 2 + 2 * 16, 2                            # ready[2] | done[2][16] | counter
    assert L.mm_p2p_set_wait_limit(1 << 27) == 0
    try:
        st.zero_()
        assert L.mm_p2p_rs(gp, fp, S, 2, 0, 0, 1, 0.5, out.data_ptr(), 0, st.data_ptr(), 8, native._st()) == 0
        torch.cuda.synchronize()
        assert int(st.item()) == 4
        assert float(out.abs().max()) == 0.0                           # the reduction was skipped
        assert flags[0, counter_idx].item() == 0                      # arrival counter is back to zero
        assert flags[1, done_idx + 0].item() == 1                     # slot handed back: done[slot 0][rank 0] = seq
        st.zero_()
        flags[1, 0] = 2                                               # the peer publishes ready[slot 0] = 2
        assert L.mm_p2p_rs(gp, fp, S, 2, 0, 0, 2, 0.5, out.data_ptr(), 0, st.data_ptr(), 8, native._st()) == 0
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        want = (g0[:S].float() + g1[:S].float()) * 0.5
        assert torch.allclose(out, want, rtol=1e-6, atol=1e-6)
        assert flags[1, done_idx + 0].item() == 2
    finally:
        assert L.mm_p2p_set_wait_limit(0) == 0
        st.zero_()
