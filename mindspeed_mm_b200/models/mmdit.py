"""Dual-stream / single-stream MMDiT family: HunyuanVideo and FLUX.

Both are "double blocks" (image and text tokens keep separate modulation, QKV and MLP weights but attend
jointly) followed by "single blocks" (one stream over the concatenation, attention and MLP computed in
parallel from one fused projection), adaLN-zero modulation from a pooled conditioning vector, QK-RMSNorm per
head and RoPE on the image tokens only (3-D (t, h, w) split for video, 2-D for FLUX).
HunyuanVideo: 20 double + 40 single blocks, 24 heads x 128, rope dims (16, 56, 56)
(mindspeed_mm/models/predictor/dits/hunyuan_video_dit.py:104-200,645,1090,1394-1560).  FLUX.1: 19 double + 38
single, 24 heads x 128, rope dims (16, 56, 56) over (id, h, w) (examples/diffusers/flux; trained natively here
instead of through diffusers scripts).  Under Ulysses only the image tokens are sequence-sharded; text tokens
are replicated and their heads are split, as the reference does for HunyuanVideo.
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
class MMDiTConfig:
    in_channels: int = 16
    out_channels: int = 16
    patch_size: Sequence[int] = (1, 2, 2)
    hidden_size: int = 3072
    num_heads: int = 24
    mlp_ratio: float = 4.0
    num_double_blocks: int = 20
    num_single_blocks: int = 40
    text_dim: int = 4096
    pooled_dim: int = 768
    rope_dims: Sequence[int] = (16, 56, 56)
    rope_theta: float = 256.0
    guidance_embed: bool = True
    eps: float = 1e-6
    init_std: float = 0.02
    # block-sparse self-attention over the latent canvas (HunyuanVideo-1.5): dict(tile=(6, 8, 8), kernel=(3, 3, 3), topk=8,
    # mode="ssta"); None = dense
    sparse_attention: Optional[dict] = None
    # HunyuanVideo: the prompt states go through a small timestep-aware transformer (the "token refiner") instead of one
    # projection; 0 = plain Linear (FLUX, SD3)
    text_refiner_layers: int = 0

    @staticmethod
    def hunyuan_video():
        return MMDiTConfig(text_refiner_layers=2)

    @staticmethod
    def hunyuan_video_15(**kw):
        """HunyuanVideo-1.5 (mindspeed_mm/models/predictor/dits/hunyuan_video_15_dit.py:698): dual-stream blocks only, 32-channel
        latents with 1 x 1 x 1 patches, selective sliding-tile attention."""
        d = dict(in_channels=32, out_channels=32, patch_size=(1, 1, 1), hidden_size=2048, num_heads=16, num_double_blocks=54,
                 num_single_blocks=0, text_dim=3584, rope_dims=(16, 56, 56), guidance_embed=False,
                 sparse_attention=dict(tile=(6, 8, 8), kernel=(3, 3, 3), topk=8, mode="ssta"))
        d.update(kw)
        return MMDiTConfig(**d)

    @staticmethod
    def flux_dev():
        return MMDiTConfig(in_channels=64, out_channels=64, patch_size=(1, 1, 1), num_double_blocks=19, num_single_blocks=38,
                           rope_theta=10000.0)

    @staticmethod
    def sd3_medium():
        """Stable Diffusion 3: dual-stream blocks only, 2x2 patches of 16-channel latents, no guidance embedding."""
        return MMDiTConfig(in_channels=16, out_channels=16, patch_size=(1, 2, 2), hidden_size=1536, num_heads=24,
                           num_double_blocks=24, num_single_blocks=0, text_dim=4096, pooled_dim=2048,
                           rope_dims=(0, 32, 32), rope_theta=10000.0, guidance_embed=False)

    @staticmethod
    def tiny():
        return MMDiTConfig(in_channels=4, out_channels=4, hidden_size=64, num_heads=4, num_double_blocks=1,
                           num_single_blocks=2, text_dim=32, pooled_dim=16, rope_dims=(4, 6, 6))


def rope_nd(grid: Tuple[int, int, int], dims: Sequence[int], theta: float, device=None):
    """cos/sin [prod(grid), sum(dims)/2] for interleaved-pair rotation; axis a uses dims[a] channels."""
    outs = []
    sizes = list(grid)
    for a, (n, d) in enumerate(zip(sizes, dims)):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=device) / d))
        ang = torch.outer(torch.arange(n, dtype=torch.float64, device=device), inv)
        shape = [1, 1, 1, d // 2]
        shape[a] = n
        outs.append(ang.view(shape).expand(*sizes, d // 2))
    ang = torch.cat(outs, -1).reshape(-1, sum(dims) // 2)
    return ang.cos().float(), ang.sin().float()


class Modulation(nn.Module):
    def __init__(self, dim, n):
        super().__init__()
        self.n = n
        self.lin = Linear(dim, n * dim)

    def forward(self, vec):                       # vec [B, H] -> n x [B, 1, H]
        return self.lin(F.silu(vec)).unsqueeze(1).chunk(self.n, dim=-1)


class StreamParams(nn.Module):
    """Per-stream weights of a double block."""

    def __init__(self, c: MMDiTConfig):
        super().__init__()
        H, nh = c.hidden_size, c.num_heads
        self.mod = Modulation(H, 6)
        self.qkv = Linear(H, 3 * H)
        self.q_norm, self.k_norm = RMSNorm(H // nh, c.eps), RMSNorm(H // nh, c.eps)
        self.proj = Linear(H, H)
        self.mlp_0 = Linear(H, int(H * c.mlp_ratio))
        self.mlp_2 = Linear(int(H * c.mlp_ratio), H)


def _heads(x, nh):
    B, S, H = x.shape
    return x.view(B, S, nh, H // nh)


def _attend(c: "MMDiTConfig", q, k, v, s_img: int, grid):
    """Joint attention over [image tokens, text tokens]; block-sparse on the image canvas when the config asks for it."""
    sp = c.sparse_attention
    if not sp or grid is None:
        return ops.attention_dense(q, k, v)
    from ..ops.sparse_attention import ssta_attention
    return ssta_attention(q, k, v, grid, tuple(sp.get("tile", (6, 8, 8))), tuple(sp.get("kernel", (1, 1, 1))), int(sp.get("topk", 1)),
                          text_len=q.shape[1] - s_img, mode=sp.get("mode", "ssta"), pad=sp.get("pad", "zero"),
                          share_heads=sp.get("share_heads", True))[0]


def _rope(x, cos, sin):
    B, S, N, D = x.shape
    return ops.rope_interleaved(x.reshape(B * S, N, D), cos.repeat(B, 1), sin.repeat(B, 1)).view(B, S, N, D)


class DoubleBlock(nn.Module):
    def __init__(self, c: MMDiTConfig):
        super().__init__()
        self.c = c
        self.img, self.txt = StreamParams(c), StreamParams(c)

    def forward(self, img, txt, vec, cos, sin, grid=None):
        c, nh = self.c, self.c.num_heads
        im, tm = self.img.mod(vec), self.txt.mod(vec)
        qkvs = []
        for x, sp, m in ((img, self.img, im), (txt, self.txt, tm)):
            h = ops.layer_norm_modulate(x, m[1], m[0], c.eps)
            q, k, v = sp.qkv(h).chunk(3, dim=-1)
            qkvs.append((sp.q_norm(_heads(q, nh)), sp.k_norm(_heads(k, nh)), _heads(v, nh)))
        (qi, ki, vi), (qt, kt, vt) = qkvs
        qi, ki = _rope(qi, cos, sin), _rope(ki, cos, sin)
        q, k, v = torch.cat([qi, qt], 1), torch.cat([ki, kt], 1), torch.cat([vi, vt], 1)
        S_img = img.shape[1]
        o = _attend(c, q, k, v, S_img, grid)
        oi, ot = o[:, :S_img].flatten(2), o[:, S_img:].flatten(2)
        outs = []
        for x, o_, sp, m in ((img, oi, self.img, im), (txt, ot, self.txt, tm)):
            x = ops.gated_residual(x, sp.proj(o_), m[2])
            y = sp.mlp_2(ops.gelu_tanh(sp.mlp_0(ops.layer_norm_modulate(x, m[4], m[3], c.eps))))
            outs.append(ops.gated_residual(x, y, m[5]))
        return outs[0], outs[1]


class SingleBlock(nn.Module):
    def __init__(self, c: MMDiTConfig):
        super().__init__()
        self.c = c
        H, nh = c.hidden_size, c.num_heads
        self.mlp_dim = int(H * c.mlp_ratio)
        self.mod = Modulation(H, 3)
        self.linear1 = Linear(H, 3 * H + self.mlp_dim)
        self.linear2 = Linear(H + self.mlp_dim, H)
        self.q_norm, self.k_norm = RMSNorm(H // nh, c.eps), RMSNorm(H // nh, c.eps)

    def forward(self, x, vec, cos, sin, s_img: int, grid=None):
        c, nh = self.c, self.c.num_heads
        m = self.mod(vec)
        h = ops.layer_norm_modulate(x, m[1], m[0], c.eps)
        qkv, mlp = self.linear1(h).split([3 * c.hidden_size, self.mlp_dim], dim=-1)
        q, k, v = qkv.chunk(3, dim=-1)
        q, k, v = self.q_norm(_heads(q, nh)), self.k_norm(_heads(k, nh)), _heads(v, nh)
        q = torch.cat([_rope(q[:, :s_img], cos, sin), q[:, s_img:]], 1)
        k = torch.cat([_rope(k[:, :s_img], cos, sin), k[:, s_img:]], 1)
        o = _attend(c, q, k, v, s_img, grid).flatten(2)
        y = self.linear2(torch.cat([o, ops.gelu_tanh(mlp)], dim=-1))
        return ops.gated_residual(x, y, m[2])


class TokenRefinerBlock(nn.Module):
    """Pre-LayerNorm self-attention + SiLU MLP over the prompt tokens, both gated by the conditioning vector."""

    def __init__(self, c: MMDiTConfig):
        super().__init__()
        H = c.hidden_size
        self.nh = c.num_heads
        self.norm1, self.norm2 = ops.LayerNorm(H, eps=c.eps), ops.LayerNorm(H, eps=c.eps)
        self.qkv, self.proj = Linear(H, 3 * H), Linear(H, H)
        self.mlp_0, self.mlp_2 = Linear(H, int(H * c.mlp_ratio)), Linear(int(H * c.mlp_ratio), H)
        self.mod = Linear(H, 2 * H)

    def forward(self, x, cvec, mask=None):
        gate_msa, gate_mlp = self.mod(F.silu(cvec)).unsqueeze(1).chunk(2, dim=-1)
        q, k, v = (_heads(t, self.nh) for t in self.qkv(self.norm1(x)).chunk(3, dim=-1))
        if mask is None:
            o = ops.attention_dense(q, k, v)
        else:       # padded prompts: a token pair attends when both are real; everybody may look at token 0
            am = mask[:, None, :, None] & mask[:, None, None, :]
            am = am.clone()
            am[..., 0] = True
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=am).transpose(1, 2)
        x = x + self.proj(o.flatten(2)) * gate_msa
        return x + self.mlp_2(F.silu(self.mlp_0(self.norm2(x)))) * gate_mlp


class TokenRefiner(nn.Module):
    """HunyuanVideo's prompt branch in front of the blocks (mindspeed_mm/models/common/embeddings/text_embeddings.py:41-260):
    the conditioning vector is ``time embedding + projection of the (masked) mean prompt state``; the prompt states are
    embedded and refined by ``layers`` gated transformer blocks."""

    def __init__(self, c: MMDiTConfig):
        super().__init__()
        H = c.hidden_size
        self.input_embedder = Linear(c.text_dim, H)
        self.t_0, self.t_2 = Linear(256, H), Linear(H, H)
        self.c_1, self.c_2 = Linear(c.text_dim, H), Linear(H, H)
        self.blocks = nn.ModuleList([TokenRefinerBlock(c) for _ in range(c.text_refiner_layers)])

    def forward(self, txt, t, mask=None):
        dt = self.input_embedder.weight.dtype
        txt = txt.to(dt)
        te = self.t_2(F.silu(self.t_0(sinusoidal_embedding(t, 256).to(dt))))
        if mask is None:
            ctx = txt.mean(dim=1)
        else:
            mf = mask.to(dt).unsqueeze(-1)
            ctx = (txt * mf).sum(dim=1) / mf.sum(dim=1)
        cvec = te + self.c_2(F.silu(self.c_1(ctx)))
        x = self.input_embedder(txt)
        for blk in self.blocks:
            x = blk(x, cvec, mask)
        return x


class MMDiTEmbed(nn.Module):
    def __init__(self, c: MMDiTConfig):
        super().__init__()
        self.c = c
        p = c.patch_size
        self.img_in = Linear(c.in_channels * p[0] * p[1] * p[2], c.hidden_size)
        self.txt_in = TokenRefiner(c) if c.text_refiner_layers > 0 else Linear(c.text_dim, c.hidden_size)
        self.time_in_0, self.time_in_2 = Linear(256, c.hidden_size), Linear(c.hidden_size, c.hidden_size)
        self.vector_in_0, self.vector_in_2 = Linear(c.pooled_dim, c.hidden_size), Linear(c.hidden_size, c.hidden_size)
        if c.guidance_embed:
            self.guidance_in_0, self.guidance_in_2 = Linear(256, c.hidden_size), Linear(c.hidden_size, c.hidden_size)

    def forward(self, tokens, txt, t, pooled, guidance=None, txt_mask=None):
        dt = self.img_in.weight.dtype
        vec = self.time_in_2(F.silu(self.time_in_0(sinusoidal_embedding(t, 256).to(dt))))
        vec = vec + self.vector_in_2(F.silu(self.vector_in_0(pooled.to(dt))))
        if self.c.guidance_embed and guidance is not None:
            vec = vec + self.guidance_in_2(F.silu(self.guidance_in_0(sinusoidal_embedding(guidance, 256).to(dt))))
        text = self.txt_in(txt, t, txt_mask) if self.c.text_refiner_layers > 0 else self.txt_in(txt.to(dt))
        return self.img_in(tokens.to(dt)), text, vec


class MMDiTFinal(nn.Module):
    def __init__(self, c: MMDiTConfig):
        super().__init__()
        self.c = c
        p = c.patch_size
        self.mod = Modulation(c.hidden_size, 2)
        self.linear = Linear(c.hidden_size, c.out_channels * p[0] * p[1] * p[2])

    def forward(self, x, vec):
        m = self.mod(vec)
        return self.linear(ops.layer_norm_modulate(x, m[1], m[0], self.c.eps))


class MMDiT(nn.Module):
    """``forward(latents [B,C,F,H,W], t [B], txt [B,L,text_dim], pooled [B,pooled_dim], guidance=None) -> velocity``."""
    config_class = MMDiTConfig

    def __init__(self, config: MMDiTConfig):
        super().__init__()
        self.config = config
        self.embed = MMDiTEmbed(config)
        self.double_blocks = nn.ModuleList([DoubleBlock(config) for _ in range(config.num_double_blocks)])
        self.single_blocks = nn.ModuleList([SingleBlock(config) for _ in range(config.num_single_blocks)])
        self.final = MMDiTFinal(config)

    def fsdp_units(self):
        return [("embed", self.embed)] + [(f"double_blocks.{i}", b) for i, b in enumerate(self.double_blocks)] + \
               [(f"single_blocks.{i}", b) for i, b in enumerate(self.single_blocks)] + [("final", self.final)]

    def forward(self, latents, t, txt, pooled, guidance=None, run=None, txt_mask=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        B, C, Fr, Hh, Ww = latents.shape
        pf, ph, pw = c.patch_size
        grid = (Fr // pf, Hh // ph, Ww // pw)
        x = latents.view(B, C, grid[0], pf, grid[1], ph, grid[2], pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, -1, C * pf * ph * pw)
        img, text, vec = run(self.embed, x, txt, t, pooled, guidance, txt_mask)
        cos, sin = rope_nd(grid, c.rope_dims, c.rope_theta, device=latents.device)
        for blk in self.double_blocks:
            img, text = run(blk, img, text, vec, cos, sin, grid)
        s_img = img.shape[1]
        h = torch.cat([img, text], 1)
        for blk in self.single_blocks:
            h = run(blk, h, vec, cos, sin, s_img, grid)
        y = run(self.final, h[:, :s_img], vec)
        y = y.view(B, grid[0], grid[1], grid[2], c.out_channels, pf, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return y.reshape(B, c.out_channels, Fr, Hh, Ww)


@model_register.register("hunyuanvideodit")
class HunyuanVideoDiT(MMDiT):
    def hf_ops(self):
        """Name map of the published HunyuanVideo transformer checkpoint (``checkpoint/hf.py: hunyuanvideo_ops``)."""
        from ..checkpoint.hf import hunyuanvideo_ops
        return hunyuanvideo_ops(self.config)


@model_register.register("hunyuanvideo15dit")
class HunyuanVideo15DiT(MMDiT):
    """HunyuanVideo-1.5: ``MMDiTConfig.hunyuan_video_15()``; attention over the canvas is block-sparse (``ops/sparse_attention.py``)."""
    pass


@model_register.register("flux")
class FluxDiT(MMDiT):
    pass


@model_register.register("sd3")
class SD3DiT(MMDiT):
    """Dual-stream-only MMDiT (the reference fine-tunes SD3 / SD3.5 through diffusers scripts,
    examples/diffusers/sd3/); same blocks with ``num_single_blocks = 0``."""
    pass
