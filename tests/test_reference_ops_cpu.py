"""Algebraic checks of the fp32 reference ops (they are the oracles for the CUDA kernels)."""
import math

import pytest
import torch
import torch.nn.functional as F

from mindspeed_mm_b200 import ops
from mindspeed_mm_b200.ops import reference as ref


def test_rms_norm_matches_torch():
    x = torch.randn(5, 64)
    w = torch.randn(64)
    assert torch.allclose(ref.rms_norm(x, w, 1e-6), F.rms_norm(x, (64,), w, 1e-6), atol=1e-5)


def test_swiglu():
    x = torch.randn(3, 16)
    assert torch.allclose(ref.swiglu(x), F.silu(x[:, :8]) * x[:, 8:], atol=1e-6)
    y = ref.swiglu(x * 100, clamp=7.0)
    assert y.abs().max() <= 7.0 * 7.0 + 1e-3


def test_rope_rotate_half_is_rotation():
    T, N, D = 7, 2, 16
    x = torch.randn(T, N, D)
    ang = torch.rand(T, D // 2) * 6
    emb = torch.cat([ang, ang], -1)
    y = ref.rope_rotate_half(x, emb.cos(), emb.sin())
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    back = ref.rope_rotate_half(y, emb.cos(), -emb.sin())
    assert torch.allclose(back, x, atol=1e-5)


def test_rope_interleaved_matches_complex():
    T, N, D = 6, 3, 16
    x = torch.randn(T, N, D)
    cos, sin = ref.rope3d_freqs((1, 2, 3), D)
    y = ref.rope_interleaved(x, cos, sin)
    xc = torch.view_as_complex(x.reshape(T, N, D // 2, 2))
    fc = torch.polar(torch.ones_like(cos), torch.atan2(sin, cos)).unsqueeze(1)
    assert torch.allclose(y, torch.view_as_real(xc * fc).flatten(-2), atol=1e-5)


def test_rope3d_split_dims():
    cos, sin = ref.rope3d_freqs((2, 3, 4), 128)
    assert cos.shape == (24, 64)           # (22 + 21 + 21) pairs
    # frame axis only changes the first 22 pairs
    assert torch.allclose(cos[0, 22:], cos[12, 22:])
    assert not torch.allclose(cos[0, :22], cos[12, :22])
    c16, _ = ref.rope3d_freqs((1, 1, 1), 16)
    assert c16.shape == (1, 8)


def test_mrope_text_equals_1d_rope():
    pos = torch.arange(10).view(1, -1).expand(3, -1)
    cos, sin = ref.mrope_cos_sin(pos, 128, 1e6, (16, 24, 24))
    inv = 1.0 / (1e6 ** (torch.arange(0, 64).float() / 64))
    f = torch.outer(torch.arange(10).float(), inv)
    assert torch.allclose(cos, torch.cat([f, f], -1).cos(), atol=1e-5)


def test_attention_varlen_vs_sdpa():
    torch.manual_seed(0)
    q = torch.randn(10, 4, 8)
    k = torch.randn(10, 2, 8)
    v = torch.randn(10, 2, 8)
    cu = torch.tensor([0, 4, 10])
    o = ref.attention_varlen(q, k, v, cu, cu, causal=True)
    for a, b in ((0, 4), (4, 10)):
        qq = q[a:b].transpose(0, 1).unsqueeze(0)
        kk = k[a:b].transpose(0, 1).repeat_interleave(2, 0).unsqueeze(0)
        vv = v[a:b].transpose(0, 1).repeat_interleave(2, 0).unsqueeze(0)
        r = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True)[0].transpose(0, 1)
        assert torch.allclose(o[a:b], r, atol=1e-5)


def test_merge_attention_states_equals_full():
    torch.manual_seed(0)
    q = torch.randn(5, 2, 8)
    k = torch.randn(12, 2, 8)
    v = torch.randn(12, 2, 8)
    cq = torch.tensor([0, 5])
    full = ref.attention_varlen(q, k, v, cq, torch.tensor([0, 12]))
    o1, l1 = ref.attention_varlen(q, k[:7], v[:7], cq, torch.tensor([0, 7]), return_lse=True)
    o2, l2 = ref.attention_varlen(q, k[7:], v[7:], cq, torch.tensor([0, 5]), return_lse=True)
    o, _ = ref.merge_attention_states(o1, l1, o2, l2)
    assert torch.allclose(o, full, atol=1e-5)


def test_chunked_linear_ce_matches_dense():
    torch.manual_seed(0)
    h = torch.randn(37, 16, requires_grad=True)
    w = torch.randn(50, 16, requires_grad=True)
    lab = torch.randint(0, 50, (37,))
    lab[::5] = -100
    loss, n = ops.linear_cross_entropy(h, w, lab, chunk=8)
    (loss / n).backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    r = F.cross_entropy(h2 @ w2.t(), lab, ignore_index=-100)
    r.backward()
    assert torch.allclose(loss / n, r, atol=1e-5)
    assert torch.allclose(h.grad, h2.grad, atol=1e-5)
    assert torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_grouped_gemm_and_grads():
    torch.manual_seed(0)
    counts = [3, 0, 5]
    x = torch.randn(8, 6, requires_grad=True)
    w = torch.randn(3, 6, 4, requires_grad=True)
    y = ops.grouped_gemm(x, w, counts)
    y.sum().backward()
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    r = torch.cat([x2[:3] @ w2[0], x2[3:] @ w2[2]])
    r.sum().backward()
    assert torch.allclose(y, r, atol=1e-5)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5) and torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_permute_unpermute_roundtrip():
    torch.manual_seed(0)
    T, k, E, H = 9, 2, 4, 5
    tok = torch.randn(T, H)
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    probs = torch.rand(T, k)
    perm, order = ref.moe_permute(tok, ids)
    sorted_e = ids.reshape(-1)[order]
    assert (sorted_e[1:] >= sorted_e[:-1]).all()
    out = ref.moe_unpermute(perm, order, probs)
    assert torch.allclose(out, tok * probs.sum(1, keepdim=True), atol=1e-5)


@pytest.mark.parametrize("T", [64, 100, 130])
def test_gdn_chunked_equals_recurrent(T):
    torch.manual_seed(0)
    B, H, K, V = 2, 2, 16, 12
    q = F.normalize(torch.randn(B, T, H, K), dim=-1)
    k = F.normalize(torch.randn(B, T, H, K), dim=-1)
    v = torch.randn(B, T, H, V)
    g = -torch.rand(B, T, H) * 0.5
    beta = torch.rand(B, T, H)
    o1, s1 = ref.gated_delta_rule_recurrent(q, k, v, g, beta)
    o2, s2 = ref.gated_delta_rule_chunked(q, k, v, g, beta, chunk=32)
    assert torch.allclose(o1, o2, atol=2e-4), (o1 - o2).abs().max()
    if T % 32 == 0:
        assert torch.allclose(s1, s2, atol=2e-4)


def test_causal_conv1d_varlen_is_causal():
    torch.manual_seed(0)
    x = torch.randn(12, 6)
    w = torch.randn(6, 4)
    y = ref.causal_conv1d(x, w, activation=None, cu_seqlens=[0, 5, 12])
    x2 = x.clone()
    x2[4] += 10.0           # last token of segment 0 must not leak into segment 1
    y2 = ref.causal_conv1d(x2, w, activation=None, cu_seqlens=[0, 5, 12])
    assert torch.allclose(y[5:], y2[5:])
    assert torch.allclose(y[:4], y2[:4])


def test_adamw_matches_torch():
    torch.manual_seed(0)
    p = torch.randn(100)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(100), torch.zeros(100)
    for step in range(1, 4):
        g = torch.randn(100)
        ref_p.grad = g.clone()
        opt.step()
        ref.adamw_step(p, m, v, g, 1e-2, 0.9, 0.999, 1e-8, 0.1, step)
    assert torch.allclose(p, ref_p.data, atol=1e-6)


def test_gdn_prologue_state_pass_and_hand_backward_match_recurrence():
    """Batched prologue + state walk + hand-written backward == autograd of the token-by-token recurrence."""
    import torch.nn.functional as F
    from mindspeed_mm_b200.ops import gdn
    torch.manual_seed(0)
    T, H, K, V = 200, 2, 128, 128
    cu = [0, 70, 200]
    q = F.normalize(torch.randn(T, H, K), dim=-1).requires_grad_()
    k = F.normalize(torch.randn(T, H, K), dim=-1).requires_grad_()
    v = torch.randn(T, H, V).requires_grad_()
    g = (-0.5 * torch.rand(T, H)).requires_grad_()
    beta = torch.rand(T, H).requires_grad_()
    o = gdn.gated_delta_rule_varlen(q, k, v, g, beta, cu)
    outs = []
    for a, b in zip(cu[:-1], cu[1:]):
        oo, _ = ref.gated_delta_rule_recurrent(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b], beta[None, a:b])
        outs.append(oo[0])
    o_ref = torch.cat(outs)
    assert torch.allclose(o, o_ref, atol=1e-5)
    do = torch.randn_like(o)
    got = torch.autograd.grad(o, [q, k, v, g, beta], do)
    want = torch.autograd.grad(o_ref, [q, k, v, g, beta], do)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()


def test_kda_chunked_matches_recurrent():
    torch.manual_seed(0)
    B, T, H, K, V = 2, 150, 2, 32, 16
    q = F.normalize(torch.randn(B, T, H, K), dim=-1)
    k = F.normalize(torch.randn(B, T, H, K), dim=-1)
    v = torch.randn(B, T, H, V)
    g = -0.1 * torch.rand(B, T, H, K)
    beta = torch.rand(B, T, H)
    o1, s1 = ref.kda_recurrent(q, k, v, g, beta)
    o2, s2 = ref.kda_chunked(q, k, v, g, beta, chunk=64)
    assert torch.allclose(o1, o2, atol=2e-4), (o1 - o2).abs().max()
    assert torch.allclose(s1, s2, atol=2e-4)


def test_kda_varlen_state_pass_and_hand_backward_match_recurrence():
    """Packed KDA (batched per-channel prologue + state walk with a decay per key channel + hand-written backward)
    == autograd of the token-by-token recurrence."""
    from mindspeed_mm_b200 import ops
    torch.manual_seed(0)
    T, H, K, V = 200, 2, 128, 128
    cu = [0, 70, 200]
    q = F.normalize(torch.randn(T, H, K), dim=-1).requires_grad_()
    k = F.normalize(torch.randn(T, H, K), dim=-1).requires_grad_()
    v = torch.randn(T, H, V).requires_grad_()
    g = (-0.1 * torch.rand(T, H, K)).requires_grad_()
    beta = torch.rand(T, H).requires_grad_()
    o = ops.kda_varlen(q, k, v, g, beta, cu)
    outs = []
    for a, b in zip(cu[:-1], cu[1:]):
        oo, _ = ref.kda_recurrent(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b], beta[None, a:b])
        outs.append(oo[0])
    o_ref = torch.cat(outs)
    assert torch.allclose(o, o_ref, atol=2e-5), (o - o_ref).abs().max()
    do = torch.randn_like(o)
    got = torch.autograd.grad(o, [q, k, v, g, beta], do)
    want = torch.autograd.grad(o_ref, [q, k, v, g, beta], do)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=5e-5), (a - b).abs().max()


# ------------------------------------------------------------------------------------------------- block-sparse attention
def test_sta_mask_window_is_clamped_at_borders():
    from mindspeed_mm_b200.ops.sparse_attention import sta_block_mask, tile_order
    m = sta_block_mask((1, 4, 4), (1, 3, 3))
    assert m.shape == (16, 16) and (m.sum(1) == 9).all()                 # every tile sees a full 3 x 3 window
    assert m[0].nonzero().flatten().tolist() == [0, 1, 2, 4, 5, 6, 8, 9, 10]     # corner tile: window shifted inwards
    assert m[5].nonzero().flatten().tolist() == [0, 1, 2, 4, 5, 6, 8, 9, 10]
    assert sta_block_mask((2, 2, 2), (3, 3, 3)).all()
    perm = tile_order((2, 4, 4), (1, 2, 2))
    assert perm[:4].tolist() == [0, 1, 4, 5] and sorted(perm.tolist()) == list(range(32))


def test_ssta_equals_dense_when_every_block_is_selected_and_is_sparse_otherwise():
    from mindspeed_mm_b200.ops import reference as R
    from mindspeed_mm_b200.ops.sparse_attention import ssta_attention
    torch.manual_seed(0)
    B, N, D = 2, 2, 16
    canvas, tile, text = (2, 4, 4), (1, 2, 2), 4
    S = 2 * 4 * 4 + text
    q, k, v = (torch.randn(B, S, N, D) for _ in range(3))
    dense = R.attention_dense(q, k, v)
    full, density = ssta_attention(q, k, v, canvas, tile, kernel=(5, 5, 5), topk=1, text_len=text)
    assert density == 1.0 and torch.allclose(full, dense, atol=1e-5)
    sparse, density = ssta_attention(q, k, v, canvas, tile, kernel=(1, 1, 1), topk=2, text_len=text)
    assert 0 < density < 1 and sparse.shape == dense.shape and not torch.allclose(sparse, dense, atol=1e-3)
    # text rows see everything in every mode
    assert torch.allclose(sparse[:, -text:], dense[:, -text:], atol=1e-5)
    # window-only mode and per-head selection run and differ from each other
    sta, d_sta = ssta_attention(q, k, v, canvas, tile, kernel=(1, 3, 3), text_len=text, mode="sta")
    per_head, _ = ssta_attention(q, k, v, canvas, tile, kernel=(1, 1, 1), topk=2, text_len=text, share_heads=False)
    assert d_sta < 1 and sta.shape == per_head.shape == dense.shape
    # a canvas that is not a multiple of the tile is padded and cropped back
    q2, k2, v2 = (torch.randn(1, 3 * 3 * 5, N, D) for _ in range(3))
    out, _ = ssta_attention(q2, k2, v2, (3, 3, 5), (2, 2, 2), kernel=(1, 1, 1), topk=1)
    assert out.shape == q2.shape and torch.isfinite(out).all()
