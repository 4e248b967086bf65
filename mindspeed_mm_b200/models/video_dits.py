"""The other diffusion transformers of the generation zoo, built from two block families.

``CrossDiT``  -- adaLN-single blocks (one time embedding projected once to 6 modulation vectors, plus a learned per-block
table): self-attention over the latent tokens with 3-D rotary positions -> cross-attention to the text tokens -> MLP.
Stands for StepVideo (mindspeed_mm/models/predictor/dits/step_video_dit.py), Open-Sora-Plan v1.3 ``VideoDitSparse`` with
"sparse 1-D" attention that splits the sequence into ``sparse_n`` interleaved or contiguous groups on alternating layers
(video_dit_sparse.py), its U-shaped variant with long skip connections (sparseu_mmdit.py), Latte / PT-DiT style
PixArt blocks (pt_dit_diffusers.py).

``JointDiT``  -- text tokens are concatenated in front of the video tokens and every block runs one joint self-attention;
layer norms are modulated separately for the two parts ("expert" adaLN).  Stands for CogVideoX (sat_dit.py).

Both return the prediction with the latent's shape ``[B, C, F, H, W]`` (twice the channels when ``learn_sigma``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .qwen2_5_vl import Linear, RMSNorm
from .registry import model_register
from .wan import sinusoidal_embedding


@dataclass
class VideoDiTConfig:
    in_channels: int = 16
    out_channels: int = 16
    patch_size: Sequence[int] = (1, 2, 2)
    hidden_size: int = 1152
    num_heads: int = 16
    num_layers: int = 28
    mlp_ratio: float = 4.0
    text_dim: int = 4096
    text_dim_2: int = 0                  # second text encoder (StepVideo: CLIP-style features projected and appended)
    freq_dim: int = 256
    qk_norm: bool = True
    rope_theta: float = 10000.0
    learn_sigma: bool = False
    sparse_n: int = 1                    # > 1: sparse 1-D attention, groups alternate between interleaved and contiguous
    sparse_1d: bool = True
    skip_connections: bool = False       # U-shaped: block i of the second half also receives block (L - 1 - i)'s output
    eps: float = 1e-6
    init_std: float = 0.02

    @staticmethod
    def step_video(**kw):
        d = dict(in_channels=64, out_channels=64, patch_size=(1, 1, 1), hidden_size=6144, num_heads=48, num_layers=48,
                 text_dim=6144, text_dim_2=1024)
        d.update(kw)
        return VideoDiTConfig(**d)

    @staticmethod
    def open_sora_plan(**kw):
        d = dict(in_channels=8, out_channels=8, patch_size=(1, 2, 2), hidden_size=2304, num_heads=24, num_layers=32, sparse_n=4)
        d.update(kw)
        return VideoDiTConfig(**d)

    @staticmethod
    def cogvideox_5b(**kw):
        d = dict(in_channels=16, out_channels=16, patch_size=(1, 2, 2), hidden_size=3072, num_heads=48, num_layers=42)
        d.update(kw)
        return VideoDiTConfig(**d)

    @staticmethod
    def tiny(**kw):
        d = dict(in_channels=4, out_channels=4, hidden_size=64, num_heads=4, num_layers=2, text_dim=32, freq_dim=32)
        d.update(kw)
        return VideoDiTConfig(**d)


class _Attention(nn.Module):
    def __init__(self, c: VideoDiTConfig, kv_dim: Optional[int] = None):
        super().__init__()
        H = c.hidden_size
        self.nh, self.hd = c.num_heads, H // c.num_heads
        self.q = Linear(H, H)
        self.kv = Linear(kv_dim or H, 2 * H)
        self.o = Linear(H, H)
        self.q_norm = RMSNorm(self.hd, c.eps) if c.qk_norm else nn.Identity()
        self.k_norm = RMSNorm(self.hd, c.eps) if c.qk_norm else nn.Identity()

    def project(self, x, ctx):
        B, S, H = x.shape
        q = self.q_norm(self.q(x).view(B, S, self.nh, self.hd))
        k, v = self.kv(ctx).view(B, ctx.shape[1], 2, self.nh, self.hd).unbind(2)
        return q, self.k_norm(k), v


def _rope(x, cos, sin):
    B, S, N, D = x.shape
    return ops.rope_interleaved(x.reshape(B * S, N, D), cos.repeat(B, 1), sin.repeat(B, 1)).view(B, S, N, D)


def sparse_1d_groups(S: int, n: int, contiguous: bool, device=None) -> torch.Tensor:
    """Index tensor [n, ceil(S / n)] assigning tokens to ``n`` attention groups (padding slots hold -1): strided
    (token i -> group i % n) or contiguous chunks."""
    per = (S + n - 1) // n
    idx = torch.full((n * per,), -1, dtype=torch.long, device=device)
    idx[:S] = torch.arange(S, device=device)
    return idx.view(n, per) if contiguous else idx.view(per, n).t().contiguous()


def grouped_self_attention(q, k, v, groups: torch.Tensor):
    """Attention restricted to the token groups of ``groups`` [n, per] (-1 = padding).  q, k, v [B, S, N, D]."""
    B, S, N, D = q.shape
    n, per = groups.shape
    valid = groups >= 0
    g = groups.clamp(min=0).reshape(-1)
    qg, kg, vg = (t[:, g].view(B, n, per, N, D).reshape(B * n, per, N, D) for t in (q, k, v))
    if bool(valid.all()):
        og = ops.attention_dense(qg, kg, vg)
    else:
        bias = torch.zeros(n, 1, 1, per, dtype=q.dtype, device=q.device).masked_fill(~valid[:, None, None], float("-inf"))
        og = F.scaled_dot_product_attention(qg.transpose(1, 2), kg.transpose(1, 2), vg.transpose(1, 2),
                                            attn_mask=bias.repeat(B, 1, 1, 1)).transpose(1, 2)
    out = torch.zeros_like(q)
    flat = og.reshape(B, n * per, N, D)
    keep = valid.reshape(-1)
    out[:, g[keep]] = flat[:, keep]
    return out


# ------------------------------------------------------------------------------------------------- adaLN-single family
class CrossBlock(nn.Module):
    def __init__(self, c: VideoDiTConfig, index: int, skip: bool = False):
        super().__init__()
        self.c, self.index = c, index
        H = c.hidden_size
        self.scale_shift_table = nn.Parameter(torch.randn(6, H) / H ** 0.5)
        self.attn1 = _Attention(c)
        self.attn2 = _Attention(c, H)
        self.ff_0, self.ff_2 = Linear(H, int(H * c.mlp_ratio)), Linear(int(H * c.mlp_ratio), H)
        self.skip_proj = Linear(2 * H, H) if skip else None

    def forward(self, x, temb6, text, text_mask, cos, sin, skip=None):
        c = self.c
        if self.skip_proj is not None and skip is not None:
            x = self.skip_proj(torch.cat([x, skip], -1))
        m = (self.scale_shift_table.to(x.dtype)[None] + temb6).unbind(1)                 # 6 x [B, H]
        m = [t[:, None] for t in m]
        h = ops.layer_norm_modulate(x, m[1], m[0], c.eps)
        q, k, v = self.attn1.project(h, h)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        if c.sparse_n > 1:
            groups = sparse_1d_groups(x.shape[1], c.sparse_n, contiguous=bool(self.index % 2) if c.sparse_1d else True, device=x.device)
            o = grouped_self_attention(q, k, v, groups)
        else:
            o = ops.attention_dense(q, k, v)
        x = ops.gated_residual(x, self.attn1.o(o.flatten(2)), m[2])
        q, k, v = self.attn2.project(x, text)
        if text_mask is None:
            o = ops.attention_dense(q, k, v)
        else:
            bias = torch.zeros(x.shape[0], 1, 1, text.shape[1], dtype=q.dtype, device=q.device)
            bias = bias.masked_fill(~text_mask.bool()[:, None, None], float("-inf"))
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=bias).transpose(1, 2)
        x = x + self.attn2.o(o.flatten(2))
        y = self.ff_2(ops.gelu_tanh(self.ff_0(ops.layer_norm_modulate(x, m[4], m[3], c.eps))))
        return ops.gated_residual(x, y, m[5])


class _Embed(nn.Module):
    def __init__(self, c: VideoDiTConfig, n_mod: int):
        super().__init__()
        self.c = c
        p = c.patch_size
        H = c.hidden_size
        self.patch = Linear(c.in_channels * p[0] * p[1] * p[2], H)
        self.t1, self.t2 = Linear(c.freq_dim, H), Linear(H, H)
        self.t_proj = Linear(H, n_mod * H)
        self.text_1, self.text_2 = Linear(c.text_dim, H), Linear(H, H)
        self.text2_proj = Linear(c.text_dim_2, H) if c.text_dim_2 else None
        self.n_mod = n_mod

    def forward(self, latents, t, text, text_2=None):
        c = self.c
        B, C, Fr, Hh, Ww = latents.shape
        pf, ph, pw = c.patch_size
        grid = (Fr // pf, Hh // ph, Ww // pw)
        tok = latents.view(B, C, grid[0], pf, grid[1], ph, grid[2], pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, -1, C * pf * ph * pw)
        x = self.patch(tok.to(self.patch.weight.dtype))
        temb = self.t2(F.silu(self.t1(sinusoidal_embedding(t, c.freq_dim).to(x.dtype))))
        mod = self.t_proj(F.silu(temb)).view(B, self.n_mod, -1)
        ctx = self.text_2(ops.gelu_tanh(self.text_1(text.to(x.dtype))))
        if self.text2_proj is not None and text_2 is not None:
            ctx = torch.cat([ctx, self.text2_proj(text_2.to(x.dtype))], 1)
        return x, temb, mod, ctx, grid


class _Final(nn.Module):
    def __init__(self, c: VideoDiTConfig):
        super().__init__()
        self.c = c
        p = c.patch_size
        self.table = nn.Parameter(torch.randn(2, c.hidden_size) / c.hidden_size ** 0.5)
        self.out_ch = c.out_channels * (2 if c.learn_sigma else 1)
        self.linear = Linear(c.hidden_size, self.out_ch * p[0] * p[1] * p[2])

    def forward(self, x, temb, grid):
        sh, sc = (self.table.to(x.dtype)[None] + temb[:, None]).unbind(1)
        y = self.linear(ops.layer_norm_modulate(x, sc[:, None], sh[:, None], self.c.eps))
        B = y.shape[0]
        pf, ph, pw = self.c.patch_size
        y = y.view(B, grid[0], grid[1], grid[2], self.out_ch, pf, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return y.reshape(B, self.out_ch, grid[0] * pf, grid[1] * ph, grid[2] * pw)


class CrossDiT(nn.Module):
    """``forward(latents [B, C, F, H, W], t [B], text [B, L, text_dim], text_mask=None, text_2=None) -> prediction``."""
    cond_input = "prompt_mask"          # which batch entry the generic training wrapper passes as the fourth argument

    def __init__(self, config: VideoDiTConfig):
        super().__init__()
        self.config = c = config
        self.embed = _Embed(c, 6)
        half = c.num_layers // 2
        self.blocks = nn.ModuleList(CrossBlock(c, i, skip=c.skip_connections and i >= c.num_layers - half)
                                    for i in range(c.num_layers))
        self.final = _Final(c)

    def fsdp_units(self):
        return [("embed", self.embed)] + [(f"blocks.{i}", b) for i, b in enumerate(self.blocks)] + [("final", self.final)]

    def forward(self, latents, t, text, text_mask=None, text_2=None, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        x, temb, mod, ctx, grid = run(self.embed, latents, t, text, text_2)
        if text_mask is not None and ctx.shape[1] != text_mask.shape[1]:
            text_mask = F.pad(text_mask, (0, ctx.shape[1] - text_mask.shape[1]), value=1)
        cos, sin = ops.ref.rope3d_freqs(grid, c.hidden_size // c.num_heads, c.rope_theta, device=x.device)
        stack = []
        L, half = c.num_layers, c.num_layers // 2
        for i, blk in enumerate(self.blocks):
            skip = stack.pop() if (c.skip_connections and i >= L - half and stack) else None
            x = run(blk, x, mod, ctx, text_mask, cos, sin, skip)
            if c.skip_connections and i < half:
                stack.append(x)
        return run(self.final, x, temb, grid)


# ------------------------------------------------------------------------------------------------- joint (CogVideoX) family
class JointBlock(nn.Module):
    def __init__(self, c: VideoDiTConfig):
        super().__init__()
        self.c = c
        H = c.hidden_size
        self.attn = _Attention(c)
        self.ff_0, self.ff_2 = Linear(H, int(H * c.mlp_ratio)), Linear(int(H * c.mlp_ratio), H)
        self.ada = Linear(H, 12 * H)                      # 6 vectors for the video tokens, 6 for the text tokens

    def _mod(self, x, n_text, sc_t, sh_t, sc_v, sh_v):
        c = self.c
        t = ops.layer_norm_modulate(x[:, :n_text], sc_t, sh_t, c.eps)
        v = ops.layer_norm_modulate(x[:, n_text:], sc_v, sh_v, c.eps)
        return torch.cat([t, v], 1)

    def forward(self, x, temb, n_text, cos, sin):
        m = [t[:, None] for t in self.ada(F.silu(temb)).chunk(12, -1)]
        sh1v, sc1v, g1v, sh2v, sc2v, g2v, sh1t, sc1t, g1t, sh2t, sc2t, g2t = m
        h = self._mod(x, n_text, sc1t, sh1t, sc1v, sh1v)
        q, k, v = self.attn.project(h, h)
        q = torch.cat([q[:, :n_text], _rope(q[:, n_text:], cos, sin)], 1)
        k = torch.cat([k[:, :n_text], _rope(k[:, n_text:], cos, sin)], 1)
        o = self.attn.o(ops.attention_dense(q, k, v).flatten(2))
        x = torch.cat([x[:, :n_text] + g1t * o[:, :n_text], x[:, n_text:] + g1v * o[:, n_text:]], 1)
        y = self.ff_2(ops.gelu_tanh(self.ff_0(self._mod(x, n_text, sc2t, sh2t, sc2v, sh2v))))
        return torch.cat([x[:, :n_text] + g2t * y[:, :n_text], x[:, n_text:] + g2v * y[:, n_text:]], 1)


class JointDiT(nn.Module):
    cond_input = "prompt_mask"

    def __init__(self, config: VideoDiTConfig):
        super().__init__()
        self.config = c = config
        self.embed = _Embed(c, 1)
        self.blocks = nn.ModuleList(JointBlock(c) for _ in range(c.num_layers))
        self.norm_final = ops.LayerNorm(c.hidden_size, eps=c.eps)
        self.final = _Final(c)

    def fsdp_units(self):
        return [("embed", self.embed)] + [(f"blocks.{i}", b) for i, b in enumerate(self.blocks)] + \
               [("norm_final", self.norm_final), ("final", self.final)]

    def forward(self, latents, t, text, text_mask=None, run=None, **_):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        x, temb, _, ctx, grid = run(self.embed, latents, t, text, None)
        n_text = ctx.shape[1]
        cos, sin = ops.ref.rope3d_freqs(grid, c.hidden_size // c.num_heads, c.rope_theta, device=x.device)
        h = torch.cat([ctx, x], 1)
        for blk in self.blocks:
            h = run(blk, h, temb, n_text, cos, sin)
        h = run(self.norm_final, h)[:, n_text:]
        return run(self.final, h, temb, grid)


def _register(name: str, cls, preset):
    def build(config=None, **kw):
        if isinstance(config, VideoDiTConfig):
            return cls(config)
        if isinstance(config, dict):
            keys = VideoDiTConfig.__dataclass_fields__.keys()
            kw = {**{k: (tuple(v) if isinstance(v, list) else v) for k, v in config.items() if k in keys}, **kw}
        return cls(preset(**kw))
    model_register.register(name)(build)


_register("stepvideodit", CrossDiT, VideoDiTConfig.step_video)
_register("videoditsparse", CrossDiT, VideoDiTConfig.open_sora_plan)
_register("videoditsparsei2v", CrossDiT, lambda **kw: VideoDiTConfig.open_sora_plan(**{"in_channels": 8 * 2 + 1, **kw}))
_register("sparseummdit", CrossDiT, lambda **kw: VideoDiTConfig.open_sora_plan(**{"skip_connections": True, **kw}))
_register("ptdit", CrossDiT, lambda **kw: VideoDiTConfig(**{"learn_sigma": True, **kw}))
_register("latte", CrossDiT, lambda **kw: VideoDiTConfig(**{"learn_sigma": True, **kw}))
_register("satdit", JointDiT, VideoDiTConfig.cogvideox_5b)
