"""Stable Diffusion XL denoiser: a text-conditioned 2-D UNet with transformer stages.

The reference fine-tunes and pre-trains SDXL through the diffusers training scripts
(examples/diffusers/sdxl/train_text_to_image_sdxl_pretrain.py: ``UNet2DConditionModel`` loaded at :738, the extra
conditioning built by ``compute_time_ids`` at :1078 and passed as ``added_cond_kwargs`` at :1131, epsilon / v-prediction
target at :1120-1128, optional min-SNR weights at :1140-1156).  The network is written out here so that it runs on this
engine: every resolution stage is one sharding unit and all attention goes through ``ops.attention_dense``.

Structure (``SDXLConfig.base()``): 4 -> 320 input convolution; three encoder stages of two residual blocks with channels
(320, 640, 1280), the 2nd and 3rd followed per block by a transformer of (2, 10) layers (self-attention, cross-attention
to the 2048-wide prompt states, GEGLU feed-forward); a middle stage; a mirrored decoder with three residual blocks per
stage that consume the encoder's skip tensors.  The time embedding is the sum of the timestep MLP and of an MLP over
[pooled prompt embedding, sinusoidal codes of (original size, crop offset, target size)].
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .registry import model_register


@dataclass
class SDXLConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_channels: Tuple[int, ...] = (320, 640, 1280)
    layers_per_block: int = 2
    transformer_layers: Tuple[int, ...] = (0, 2, 10)          # per stage; 0 = plain residual stage
    head_dim: int = 64
    cross_dim: int = 2048
    pooled_dim: int = 1280
    time_id_dim: int = 256                                    # sinusoidal width of each of the 6 size / crop numbers
    num_time_ids: int = 6
    groups: int = 32
    prediction_type: str = "epsilon"

    @classmethod
    def base(cls, **kw):
        return cls(**kw)

    @classmethod
    def tiny(cls, **kw):
        d = dict(block_channels=(32, 64), transformer_layers=(0, 1), head_dim=16, cross_dim=48, pooled_dim=24,
                 time_id_dim=8, groups=8)
        d.update(kw)
        return cls(**d)

    @property
    def time_dim(self) -> int:
        return self.block_channels[0] * 4

    @property
    def text_dim(self) -> int:
        return self.cross_dim


def sinusoid(t: torch.Tensor, dim: int, flip: bool = True, shift: float = 0.0) -> torch.Tensor:
    """t [...] -> [..., dim]; (cos, sin) order when ``flip`` (the SD convention)."""
    half = dim // 2
    freq = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / (half - shift))
    a = t.float()[..., None] * freq
    return torch.cat([a.cos(), a.sin()] if flip else [a.sin(), a.cos()], -1)


class ResBlock(nn.Module):
    def __init__(self, cin, cout, tdim, groups):
        super().__init__()
        self.norm1 = nn.GroupNorm(groups, cin, eps=1e-5)
        self.conv1 = nn.Conv2d(cin, cout, 3, padding=1)
        self.time = nn.Linear(tdim, cout)
        self.norm2 = nn.GroupNorm(groups, cout, eps=1e-5)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1)
        self.skip = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x, emb):
        h = self.conv1(F.silu(self.norm1(x)))
        h = h + self.time(F.silu(emb))[:, :, None, None].to(h.dtype)
        h = self.conv2(F.silu(self.norm2(h)))
        return h + (x if self.skip is None else self.skip(x))


class Attention(nn.Module):
    def __init__(self, dim, ctx_dim, head_dim):
        super().__init__()
        self.heads = dim // head_dim
        self.to_q = nn.Linear(dim, dim, bias=False)
        self.to_k = nn.Linear(ctx_dim, dim, bias=False)
        self.to_v = nn.Linear(ctx_dim, dim, bias=False)
        self.to_out = nn.Linear(dim, dim)

    def forward(self, x, ctx=None):
        ctx = x if ctx is None else ctx
        B, S, C = x.shape
        q = self.to_q(x).view(B, S, self.heads, -1)
        k = self.to_k(ctx).view(B, ctx.shape[1], self.heads, -1)
        v = self.to_v(ctx).view(B, ctx.shape[1], self.heads, -1)
        return self.to_out(ops.attention_dense(q, k, v).reshape(B, S, C))


class TransformerLayer(nn.Module):
    def __init__(self, dim, ctx_dim, head_dim):
        super().__init__()
        self.norm1, self.norm2, self.norm3 = ops.LayerNorm(dim), ops.LayerNorm(dim), ops.LayerNorm(dim)
        self.attn1 = Attention(dim, dim, head_dim)
        self.attn2 = Attention(dim, ctx_dim, head_dim)
        self.ff_in = nn.Linear(dim, dim * 8)                   # GEGLU: value and gate halves
        self.ff_out = nn.Linear(dim * 4, dim)

    def forward(self, x, ctx):
        x = x + self.attn1(self.norm1(x))
        x = x + self.attn2(self.norm2(x), ctx)
        a, g = self.ff_in(self.norm3(x)).chunk(2, -1)
        return x + self.ff_out(a * ops.gelu(g))


class SpatialTransformer(nn.Module):
    def __init__(self, dim, ctx_dim, head_dim, depth, groups):
        super().__init__()
        self.norm = nn.GroupNorm(groups, dim, eps=1e-6)
        self.proj_in = nn.Linear(dim, dim)
        self.layers = nn.ModuleList([TransformerLayer(dim, ctx_dim, head_dim) for _ in range(depth)])
        self.proj_out = nn.Linear(dim, dim)

    def forward(self, x, ctx):
        B, C, H, W = x.shape
        h = self.proj_in(self.norm(x).flatten(2).transpose(1, 2))
        for layer in self.layers:
            h = layer(h, ctx)
        return x + self.proj_out(h).transpose(1, 2).reshape(B, C, H, W)


class Stem(nn.Module):
    """Input convolution and the two embedding MLPs; returns (features, embedding)."""

    def __init__(self, c: SDXLConfig):
        super().__init__()
        self.c = c
        ch, td = c.block_channels[0], c.time_dim
        self.conv_in = nn.Conv2d(c.in_channels, ch, 3, padding=1)
        self.time_1, self.time_2 = nn.Linear(ch, td), nn.Linear(td, td)
        add_in = c.pooled_dim + c.num_time_ids * c.time_id_dim
        self.add_1, self.add_2 = nn.Linear(add_in, td), nn.Linear(td, td)

    def forward(self, x, t, pooled, time_ids):
        c = self.c
        dt = self.time_1.weight.dtype
        emb = self.time_2(F.silu(self.time_1(sinusoid(t, c.block_channels[0]).to(dt))))
        ids = sinusoid(time_ids.reshape(-1), c.time_id_dim).reshape(time_ids.shape[0], -1)
        add = torch.cat([pooled.to(dt), ids.to(dt)], -1)
        emb = emb + self.add_2(F.silu(self.add_1(add)))
        return self.conv_in(x), emb


class DownStage(nn.Module):
    """``layers`` x (residual block [+ transformer]) and an optional stride-2 convolution; returns the output followed by
    every intermediate tensor the decoder will concatenate."""

    def __init__(self, c: SDXLConfig, cin, cout, depth, down: bool):
        super().__init__()
        self.res = nn.ModuleList([ResBlock(cin if i == 0 else cout, cout, c.time_dim, c.groups) for i in range(c.layers_per_block)])
        self.attn = nn.ModuleList([SpatialTransformer(cout, c.cross_dim, c.head_dim, depth, c.groups)
                                   for _ in range(c.layers_per_block)]) if depth else None
        self.down = nn.Conv2d(cout, cout, 3, stride=2, padding=1) if down else None

    def forward(self, x, emb, ctx):
        skips = []
        for i, r in enumerate(self.res):
            x = r(x, emb)
            if self.attn is not None:
                x = self.attn[i](x, ctx)
            skips.append(x)
        if self.down is not None:
            x = self.down(x)
            skips.append(x)
        return (x, *skips)


class MidStage(nn.Module):
    def __init__(self, c: SDXLConfig):
        super().__init__()
        ch = c.block_channels[-1]
        self.res1 = ResBlock(ch, ch, c.time_dim, c.groups)
        self.attn = SpatialTransformer(ch, c.cross_dim, c.head_dim, c.transformer_layers[-1], c.groups) \
            if c.transformer_layers[-1] else None
        self.res2 = ResBlock(ch, ch, c.time_dim, c.groups)

    def forward(self, x, emb, ctx):
        x = self.res1(x, emb)
        if self.attn is not None:
            x = self.attn(x, ctx)
        return self.res2(x, emb)


class UpStage(nn.Module):
    def __init__(self, c: SDXLConfig, cprev, cout, skip_channels: Sequence[int], depth, up: bool):
        super().__init__()
        self.res = nn.ModuleList()
        for i, cs in enumerate(skip_channels):
            self.res.append(ResBlock((cprev if i == 0 else cout) + cs, cout, c.time_dim, c.groups))
        self.attn = nn.ModuleList([SpatialTransformer(cout, c.cross_dim, c.head_dim, depth, c.groups)
                                   for _ in skip_channels]) if depth else None
        self.up = nn.Conv2d(cout, cout, 3, padding=1) if up else None

    def forward(self, x, emb, ctx, *skips):
        """``skips`` in the order they are consumed (last produced first)."""
        for i, r in enumerate(self.res):
            x = r(torch.cat([x, skips[i]], 1), emb)
            if self.attn is not None:
                x = self.attn[i](x, ctx)
        if self.up is not None:
            x = self.up(F.interpolate(x, scale_factor=2.0, mode="nearest"))
        return x


class Head(nn.Module):
    def __init__(self, c: SDXLConfig):
        super().__init__()
        self.norm = nn.GroupNorm(c.groups, c.block_channels[0], eps=1e-5)
        self.conv = nn.Conv2d(c.block_channels[0], c.out_channels, 3, padding=1)

    def forward(self, x):
        return self.conv(F.silu(self.norm(x)))


@model_register.register("sdxl_unet")
class SDXLUNet(nn.Module):
    """``forward(latents [B,C,H,W] or [B,C,1,H,W], t [B], prompt [B,L,cross_dim], added [B, pooled_dim + 6]) -> noise or
    velocity prediction`` of the latents' shape.  ``added`` = pooled prompt embedding followed by (original h, w, crop
    top, left, target h, w)."""
    config_class = SDXLConfig
    cond_input = "added_cond"

    def __init__(self, config: SDXLConfig):
        super().__init__()
        c = self.config = config
        n = len(c.block_channels)
        self.stem = Stem(c)
        self.down = nn.ModuleList()
        skip_ch: List[int] = [c.block_channels[0]]
        cin = c.block_channels[0]
        for i, ch in enumerate(c.block_channels):
            self.down.append(DownStage(c, cin, ch, c.transformer_layers[i], down=i < n - 1))
            skip_ch += [ch] * c.layers_per_block + ([ch] if i < n - 1 else [])
            cin = ch
        self.mid = MidStage(c)
        self.up = nn.ModuleList()
        self._up_counts = []
        cprev = c.block_channels[-1]
        for i in reversed(range(n)):
            take = [skip_ch.pop() for _ in range(c.layers_per_block + 1)]
            self.up.append(UpStage(c, cprev, c.block_channels[i], take, c.transformer_layers[i], up=i > 0))
            self._up_counts.append(len(take))
            cprev = c.block_channels[i]
        self.head = Head(c)

    def fsdp_units(self):
        return [("stem", self.stem)] + [(f"down.{i}", m) for i, m in enumerate(self.down)] + [("mid", self.mid)] + \
               [(f"up.{i}", m) for i, m in enumerate(self.up)] + [("head", self.head)]

    def forward(self, latents, t, prompt, added, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        video = latents.dim() == 5
        x = latents.squeeze(2) if video else latents
        pooled, time_ids = added[:, : c.pooled_dim], added[:, c.pooled_dim:]
        x, emb = run(self.stem, x, t, pooled, time_ids)
        skips = [x]
        for stage in self.down:
            x, *s = run(stage, x, emb, prompt)
            skips += s
        x = run(self.mid, x, emb, prompt)
        for stage, cnt in zip(self.up, self._up_counts):
            take = [skips.pop() for _ in range(cnt)]
            x = run(stage, x, emb, prompt, *take)
        y = run(self.head, x)
        return y.unsqueeze(2) if video else y


def compute_time_ids(original_size: Sequence[int], crop_top_left: Sequence[int], target_size: Sequence[int],
                     device=None, dtype=torch.float32) -> torch.Tensor:
    """The six size-conditioning numbers of one sample, in the order the network was trained with."""
    return torch.tensor([*original_size, *crop_top_left, *target_size], device=device, dtype=dtype)
