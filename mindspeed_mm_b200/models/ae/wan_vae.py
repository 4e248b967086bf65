"""Wan 2.1 video VAE: causal 3-D convolutional autoencoder, 4x temporal and 8x8 spatial compression, 16 latent channels.

The reference instantiates diffusers' ``AutoencoderKLWan`` behind ``AEModel`` (mindspeed_mm/models/ae/base.py:30,
mindspeed_mm/models/ae/wan_video_vae.py) and uses it frozen: ``encode`` video -> normalised latents before
``q_sample``, ``decode`` in the inference pipeline.  This file writes the network out:

* every 3-D convolution is causal in time (all temporal padding in front), so frame ``t`` of the output depends
  on frames ``<= t`` only and a video of ``1 + 4k`` frames maps to ``1 + k`` latent frames;
* the encoder is ``conv_in -> [ResBlocks (+ per-frame attention) -> Downsample] x 3 -> mid(Res, Attn, Res) -> head``;
  temporal down-sampling (stride-2 causal conv over time) happens in the last two stages; the decoder mirrors it
  with nearest-neighbour spatial up-sampling and a channel-doubling causal conv that interleaves two frames;
* latents are standardised per channel with fixed ``latents_mean / latents_std``.

Long videos are processed in temporal chunks that carry the causal-conv history (``chunk_frames``): because all
temporal context is causal the chunked result equals the one-shot result, and activation memory stays bounded.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

WAN_LATENTS_MEAN = [-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508,
                    0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921]
WAN_LATENTS_STD = [2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743,
                   3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160]


@dataclass
class WanVAEConfig:
    base_dim: int = 96
    z_dim: int = 16
    dim_mult: Sequence[int] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    attn_scales: Sequence[float] = ()
    temporal_downsample: Sequence[bool] = (False, True, True)
    in_channels: int = 3
    latents_mean: Sequence[float] = field(default_factory=lambda: list(WAN_LATENTS_MEAN))
    latents_std: Sequence[float] = field(default_factory=lambda: list(WAN_LATENTS_STD))

    @classmethod
    def tiny(cls, **kw):
        base = dict(base_dim=8, z_dim=4, dim_mult=(1, 2, 2, 2), num_res_blocks=1, latents_mean=[0.0] * 4, latents_std=[1.0] * 4)
        return cls(**{**base, **kw})


class CausalConv3d(nn.Conv3d):
    """Conv3d whose temporal padding sits entirely in front.  ``cache`` (the last ``2 * pad_t`` input frames of the
    previous chunk) replaces the zero padding when a video is processed chunk by chunk."""

    def __init__(self, cin, cout, kernel, stride=1, padding=0):
        k = (kernel,) * 3 if isinstance(kernel, int) else tuple(kernel)
        p = (padding,) * 3 if isinstance(padding, int) else tuple(padding)
        super().__init__(cin, cout, k, stride=stride, padding=0)
        self.t_pad = 2 * p[0]
        self.sp_pad = (p[2], p[2], p[1], p[1])

    def forward(self, x, cache: Optional[torch.Tensor] = None):
        t_pad = self.t_pad
        if cache is not None and t_pad > 0:
            x = torch.cat([cache[:, :, -t_pad:].to(x.dtype), x], dim=2)
            t_pad -= min(t_pad, cache.shape[2])
        x = F.pad(x, self.sp_pad + (t_pad, 0))
        return super().forward(x)


class ChannelRMSNorm(nn.Module):
    """L2-normalise over the channel dim and scale by ``sqrt(C) * gamma`` (channels-first)."""

    def __init__(self, dim, images: bool = False):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones((dim, 1, 1) if images else (dim, 1, 1, 1)))
        self.scale = dim ** 0.5

    def forward(self, x):
        return F.normalize(x.float(), dim=1).to(x.dtype) * self.scale * self.gamma


class _Cache:
    """Per-layer causal history while streaming chunks through the network (layers are visited in a fixed order)."""

    def __init__(self):
        self.slots: List[Optional[torch.Tensor]] = []
        self.i = 0

    def begin(self):
        self.i = 0

    def peek(self):
        if self.i == len(self.slots):
            self.slots.append(None)
        return self.slots[self.i]

    def push(self, value):
        self.peek()
        self.slots[self.i] = value
        self.i += 1

    def step(self, conv: "CausalConv3d", x):
        """Run ``conv`` on ``x`` with its stored history and remember the last two input frames."""
        prev = self.peek()
        tail = x[:, :, -2:].detach()
        if prev is not None and tail.shape[2] < 2:
            tail = torch.cat([prev[:, :, -(2 - tail.shape[2]):], tail], dim=2)
        y = conv(x, prev)
        self.push(tail)
        return y


def _conv(conv: CausalConv3d, x, cache: Optional[_Cache]):
    return conv(x) if cache is None else cache.step(conv, x)


class ResidualBlock(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.norm1 = ChannelRMSNorm(cin)
        self.conv1 = CausalConv3d(cin, cout, 3, padding=1)
        self.norm2 = ChannelRMSNorm(cout)
        self.conv2 = CausalConv3d(cout, cout, 3, padding=1)
        self.shortcut = CausalConv3d(cin, cout, 1) if cin != cout else None

    def forward(self, x, cache=None):
        h = self.shortcut(x) if self.shortcut is not None else x
        x = _conv(self.conv1, F.silu(self.norm1(x)), cache)
        x = _conv(self.conv2, F.silu(self.norm2(x)), cache)
        return x + h


class FrameAttention(nn.Module):
    """Single-head self-attention over the pixels of each frame."""

    def __init__(self, dim):
        super().__init__()
        self.norm = ChannelRMSNorm(dim, images=True)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
        self.proj = nn.Conv2d(dim, dim, 1)

    def forward(self, x, cache=None):
        B, C, T, H, W = x.shape
        y = x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        q, k, v = self.to_qkv(self.norm(y)).reshape(B * T, 1, 3 * C, H * W).transpose(-1, -2).chunk(3, dim=-1)
        o = F.scaled_dot_product_attention(q, k, v)
        o = self.proj(o.squeeze(1).transpose(-1, -2).reshape(B * T, C, H, W))
        return x + o.view(B, T, C, H, W).permute(0, 2, 1, 3, 4)


class Resample(nn.Module):
    """``down2d / down3d``: stride-2 spatial conv (+ stride-2 causal temporal conv); ``up2d / up3d``: nearest 2x
    spatial up-sampling + conv halving the channels (+ a causal conv that emits two frames per input frame)."""

    def __init__(self, dim, mode: str):
        super().__init__()
        self.mode = mode
        if mode.startswith("up"):
            self.spatial = nn.Conv2d(dim, dim // 2, 3, padding=1)
            self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0)) if mode == "up3d" else None
        else:
            self.spatial = nn.Conv2d(dim, dim, 3, stride=2)
            self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0)) if mode == "down3d" else None

    def _spatial(self, x):
        B, C, T, H, W = x.shape
        y = x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        if self.mode.startswith("up"):
            y = F.interpolate(y.float(), scale_factor=2.0, mode="nearest-exact").to(x.dtype)
        else:
            y = F.pad(y, (0, 1, 0, 1))
        y = self.spatial(y)
        return y.view(B, T, *y.shape[1:]).permute(0, 2, 1, 3, 4)

    def forward(self, x, cache=None, first_chunk: bool = True):
        B, C, T, H, W = x.shape
        if self.mode == "up3d":
            # the first frame of a video stays single; every later frame becomes two.  The frame-doubling conv sees
            # only the later frames (zero history in front of frame 1).
            head, rest = (x[:, :, :1], x[:, :, 1:]) if first_chunk else (x[:, :, :0], x)
            outs = [head] if head.shape[2] else []
            if rest.shape[2]:
                y = self.time_conv(rest) if cache is None else cache.step(self.time_conv, rest)
                y = y.view(B, 2, C, rest.shape[2], H, W)
                outs.append(torch.stack((y[:, 0], y[:, 1]), dim=3).reshape(B, C, rest.shape[2] * 2, H, W))
            elif cache is not None:
                cache.push(cache.peek())
            x = torch.cat(outs, dim=2) if len(outs) > 1 else outs[0]
        x = self._spatial(x)
        if self.mode == "down3d":
            # the first frame passes through; a stride-2 window of three frames (history = the previous frame,
            # frame 0 included) then halves the rest
            if cache is None or first_chunk:
                outs = [x[:, :, :1]] + ([self.time_conv(x)] if x.shape[2] >= 3 else [])
                if cache is not None:
                    cache.push(x[:, :, -1:].detach())
                x = torch.cat(outs, dim=2) if len(outs) > 1 else outs[0]
            else:
                prev = cache.peek()
                cache.push(x[:, :, -1:].detach())
                x = self.time_conv(torch.cat([prev.to(x.dtype), x], dim=2))
        return x


class Encoder3d(nn.Module):
    def __init__(self, c: WanVAEConfig):
        super().__init__()
        dims = [c.base_dim * m for m in (1,) + tuple(c.dim_mult)]
        self.conv_in = CausalConv3d(c.in_channels, dims[0], 3, padding=1)
        layers: List[nn.Module] = []
        scale = 1.0
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(c.num_res_blocks):
                layers.append(ResidualBlock(cin, cout))
                if scale in c.attn_scales:
                    layers.append(FrameAttention(cout))
                cin = cout
            if i != len(c.dim_mult) - 1:
                layers.append(Resample(cout, "down3d" if c.temporal_downsample[i] else "down2d"))
                scale /= 2.0
        self.down = nn.ModuleList(layers)
        self.mid = nn.ModuleList([ResidualBlock(dims[-1], dims[-1]), FrameAttention(dims[-1]), ResidualBlock(dims[-1], dims[-1])])
        self.norm_out = ChannelRMSNorm(dims[-1])
        self.conv_out = CausalConv3d(dims[-1], c.z_dim * 2, 3, padding=1)

    def forward(self, x, cache=None, first_chunk=True):
        x = _conv(self.conv_in, x, cache)
        for layer in list(self.down) + list(self.mid):
            x = layer(x, cache, first_chunk) if isinstance(layer, Resample) else layer(x, cache)
        return _conv(self.conv_out, F.silu(self.norm_out(x)), cache)


class Decoder3d(nn.Module):
    def __init__(self, c: WanVAEConfig):
        super().__init__()
        mult = tuple(c.dim_mult)
        dims = [c.base_dim * m for m in (mult[-1],) + mult[::-1]]
        temporal_up = tuple(c.temporal_downsample)[::-1]
        self.conv_in = CausalConv3d(c.z_dim, dims[0], 3, padding=1)
        self.mid = nn.ModuleList([ResidualBlock(dims[0], dims[0]), FrameAttention(dims[0]), ResidualBlock(dims[0], dims[0])])
        layers: List[nn.Module] = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            if i in (1, 2, 3):
                cin = cin // 2            # the preceding up-sampler halved the channels
            for _ in range(c.num_res_blocks + 1):
                layers.append(ResidualBlock(cin, cout))
                cin = cout
            if i != len(mult) - 1:
                layers.append(Resample(cout, "up3d" if temporal_up[i] else "up2d"))
        self.up = nn.ModuleList(layers)
        self.norm_out = ChannelRMSNorm(dims[-1])
        self.conv_out = CausalConv3d(dims[-1], c.in_channels, 3, padding=1)

    def forward(self, z, cache=None, first_chunk=True):
        x = _conv(self.conv_in, z, cache)
        for layer in list(self.mid) + list(self.up):
            x = layer(x, cache, first_chunk) if isinstance(layer, Resample) else layer(x, cache)
        return _conv(self.conv_out, F.silu(self.norm_out(x)), cache)


class WanVAE(nn.Module):
    """``encode(video [B,3,1+4k,H,W] in [-1,1]) -> latents [B,16,1+k,H/8,W/8]`` (standardised); ``decode`` inverts."""

    def __init__(self, c: Optional[WanVAEConfig] = None):
        super().__init__()
        self.c = c = c or WanVAEConfig()
        self.encoder = Encoder3d(c)
        self.quant_conv = CausalConv3d(c.z_dim * 2, c.z_dim * 2, 1)
        self.post_quant_conv = CausalConv3d(c.z_dim, c.z_dim, 1)
        self.decoder = Decoder3d(c)
        self.register_buffer("latents_mean", torch.tensor(list(c.latents_mean)).view(1, -1, 1, 1, 1), persistent=False)
        self.register_buffer("latents_std", torch.tensor(list(c.latents_std)).view(1, -1, 1, 1, 1), persistent=False)

    @property
    def compression(self) -> Tuple[int, int, int]:
        return (2 ** sum(self.c.temporal_downsample), 2 ** (len(self.c.dim_mult) - 1), 2 ** (len(self.c.dim_mult) - 1))

    def _moments(self, video, chunk_frames: Optional[int]):
        T = video.shape[2]
        if chunk_frames is None or T <= 1:
            return self.quant_conv(self.encoder(video))
        # first chunk: 1 frame; later chunks: multiples of the temporal compression
        step = max(self.compression[0], chunk_frames - chunk_frames % self.compression[0])
        cache = _Cache()
        outs = []
        bounds = [0, 1] + list(range(1 + step, T, step)) + [T]
        bounds = sorted(set(b for b in bounds if b <= T))
        for i, (a, b) in enumerate(zip(bounds[:-1], bounds[1:])):
            cache.begin()
            outs.append(self.encoder(video[:, :, a:b], cache, first_chunk=(i == 0)))
        return self.quant_conv(torch.cat(outs, dim=2))

    @torch.no_grad()
    def encode(self, video, sample: bool = False, generator=None, chunk_frames: Optional[int] = None):
        mean, logvar = self._moments(video, chunk_frames).chunk(2, dim=1)
        z = mean
        if sample:
            z = mean + torch.exp(0.5 * logvar.clamp(-30.0, 20.0)) * torch.randn(mean.shape, generator=generator,
                                                                                   device=mean.device, dtype=mean.dtype)
        return (z - self.latents_mean.to(z.dtype)) / self.latents_std.to(z.dtype)

    @torch.no_grad()
    def decode(self, latents, chunk_frames: Optional[int] = None):
        z = latents * self.latents_std.to(latents.dtype) + self.latents_mean.to(latents.dtype)
        z = self.post_quant_conv(z)
        if chunk_frames is None or z.shape[2] <= 1:
            return self.decoder(z).clamp(-1.0, 1.0)
        cache = _Cache()
        outs = []
        step = max(1, chunk_frames)
        bounds = sorted(set([0, 1] + list(range(1 + step, z.shape[2], step)) + [z.shape[2]]))
        for i, (a, b) in enumerate(zip(bounds[:-1], bounds[1:])):
            cache.begin()
            outs.append(self.decoder(z[:, :, a:b], cache, first_chunk=(i == 0)))
        return torch.cat(outs, dim=2).clamp(-1.0, 1.0)
