"""KL / VQ autoencoders of the generation zoo besides Wan's: one block library, four assemblies.

* ``AutoencoderKL2D``  -- image VAE (FLUX / SD3 / SD: mindspeed_mm/models/ae/flux_vae.py:12, diffusers_ae_model.py): ResNet
  stages with GroupNorm, one attention block in the middle, x8 spatial compression, ``scale_factor * (z - shift_factor)``
  latents.
* ``CausalVAE3D``      -- video VAE with causal temporal convolutions (Open-Sora-Plan ``CausalVAE`` casualvae.py:41,
  HunyuanVideo ``AutoencoderKLHunyuanVideo`` autoencoder_kl_hunyuanvideo.py, StepVideo): the first frame is
  encoded as an image, every later group of ``time_compression`` frames becomes one latent frame; spatial tiling with
  linear blending of overlaps and temporal tiling in latent-aligned chunks.
* ``WFVAE``            -- wavelet-flow VAE (wfvae.py:378): a 3-D Haar transform replaces the first down-sampling stages and the
  low-frequency band of deeper wavelet levels is injected into the encoder (and predicted by the decoder) as an
  "energy flow" side path.
* ``MOVQ``             -- vector-quantised image tokenizer (movqvae.py:12): encoder + nearest-codebook lookup, returning code
  indices for autoregressive image-token models.

All convolutions run channels-last-3d friendly shapes ``[B, C, T, H, W]``; images are ``T = 1``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------- blocks
class DiagonalGaussian:
    def __init__(self, moments: torch.Tensor, dim: int = 1):
        self.mean, logvar = moments.chunk(2, dim=dim)
        self.logvar = logvar.clamp(-30.0, 20.0)

    def sample(self, generator=None):
        noise = torch.randn(self.mean.shape, generator=generator, device=self.mean.device if generator is None else generator.device,
                            dtype=torch.float32).to(self.mean.device, self.mean.dtype)
        return self.mean + torch.exp(0.5 * self.logvar) * noise

    def mode(self):
        return self.mean

    def kl(self):
        return 0.5 * (self.mean.float() ** 2 + self.logvar.float().exp() - 1.0 - self.logvar.float()).flatten(1).sum(1)


class Conv(nn.Module):
    """3-D convolution whose temporal padding is causal (all of it in front, replicating the first frame) when the
    temporal kernel is > 1; ``spatial_only`` modules ignore time (kernel 1 along T)."""

    def __init__(self, cin, cout, k=3, stride=(1, 1, 1), causal: bool = True, kt: Optional[int] = None):
        super().__init__()
        kt = k if kt is None else kt
        self.kt, self.causal = kt, causal
        self.conv = nn.Conv3d(cin, cout, (kt, k, k), stride=stride, padding=(0, k // 2, k // 2))

    def forward(self, x):
        if self.kt > 1:
            front = self.kt - 1 if self.causal else (self.kt - 1) // 2
            back = 0 if self.causal else self.kt - 1 - front
            x = torch.cat([x[:, :, :1].expand(-1, -1, front, -1, -1), x] + ([x[:, :, -1:].expand(-1, -1, back, -1, -1)] if back else []), 2)
        return self.conv(x)


def _norm(c, groups=32):
    g = min(groups, c)
    while c % g:
        g -= 1
    return nn.GroupNorm(g, c, eps=1e-6)


class ResBlock(nn.Module):
    def __init__(self, cin, cout, kt=3):
        super().__init__()
        self.n1, self.c1 = _norm(cin), Conv(cin, cout, kt=kt)
        self.n2, self.c2 = _norm(cout), Conv(cout, cout, kt=kt)
        self.skip = Conv(cin, cout, k=1, kt=1) if cin != cout else None

    def forward(self, x):
        h = self.c1(F.silu(self.n1(x)))
        h = self.c2(F.silu(self.n2(h)))
        return (x if self.skip is None else self.skip(x)) + h


class SpatialAttention(nn.Module):
    """Single-head attention over the H x W positions of every frame."""

    def __init__(self, c):
        super().__init__()
        self.norm = _norm(c)
        self.qkv, self.proj = nn.Linear(c, 3 * c), nn.Linear(c, c)

    def forward(self, x):
        B, C, T, H, W = x.shape
        h = self.norm(x).permute(0, 2, 3, 4, 1).reshape(B * T, H * W, C)
        q, k, v = self.qkv(h).chunk(3, -1)
        o = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
        return x + self.proj(o).reshape(B, T, H, W, C).permute(0, 4, 1, 2, 3)


class Down(nn.Module):
    """Stride-2 convolution: spatial pad (0, 1) on the far sides as in the latent-diffusion encoders; with ``time`` the
    temporal stride is 2 too, with a causal front pad, so 1 + 2m frames become 1 + m."""

    def __init__(self, c, time: bool, kt=3):
        super().__init__()
        self.kt = kt if time else 1
        self.conv = nn.Conv3d(c, c, (self.kt, 3, 3), stride=(2 if time else 1, 2, 2))

    def forward(self, x):
        x = F.pad(x, (0, 1, 0, 1))
        if self.kt > 1:
            x = torch.cat([x[:, :, :1].expand(-1, -1, self.kt - 1, -1, -1), x], 2)
        return self.conv(x)


class Up(nn.Module):
    def __init__(self, c, time: bool, kt=3):
        super().__init__()
        self.time = time
        self.conv = Conv(c, c, kt=kt if time else 1)

    def forward(self, x):
        B, C, T, H, W = x.shape
        if self.time and T > 1:
            # the first latent frame stands for one pixel frame, every other one for two
            first, rest = x[:, :, :1], x[:, :, 1:]
            rest = rest.repeat_interleave(2, 2)
            x = torch.cat([first, rest], 2)
        x = F.interpolate(x.flatten(1, 2).reshape(B, C * x.shape[2], H, W), scale_factor=2.0, mode="nearest").reshape(B, C, -1, 2 * H, 2 * W)
        return self.conv(x)


# ------------------------------------------------------------------------------------------------- encoder / decoder
@dataclass
class KLVAEConfig:
    in_channels: int = 3
    out_channels: int = 3
    base: int = 128
    ch_mult: Sequence[int] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    z_channels: int = 16
    temporal_down: Sequence[bool] = (False, False, False)        # one flag per down-sampling stage
    kt: int = 3                                                   # temporal kernel (1 = pure image VAE)
    mid_attention: bool = True
    scale_factor: float = 1.0
    shift_factor: float = 0.0
    double_z: bool = True

    @classmethod
    def flux(cls, **kw):
        return cls(z_channels=16, scale_factor=0.3611, shift_factor=0.1159, kt=1, **kw)

    @classmethod
    def sd3(cls, **kw):
        return cls(z_channels=16, scale_factor=1.5305, shift_factor=0.0609, kt=1, **kw)

    @classmethod
    def sd(cls, **kw):
        return cls(z_channels=4, scale_factor=0.18215, kt=1, **kw)

    @classmethod
    def hunyuan_video(cls, **kw):
        return cls(z_channels=16, temporal_down=(False, True, True), scale_factor=0.476986, **kw)

    @classmethod
    def open_sora_plan(cls, **kw):
        return cls(z_channels=8, temporal_down=(False, True, True), ch_mult=(1, 2, 4, 4), **kw)

    @classmethod
    def tiny(cls, **kw):
        d = dict(base=16, ch_mult=(1, 2, 2), num_res_blocks=1, z_channels=4, temporal_down=(True, True))
        d.update(kw)
        return cls(**d)

    @property
    def spatial_compression(self) -> int:
        return 2 ** (len(self.ch_mult) - 1)

    @property
    def time_compression(self) -> int:
        return 2 ** sum(bool(t) for t in self.temporal_down) if self.kt > 1 else 1


class Encoder(nn.Module):
    def __init__(self, c: KLVAEConfig, in_channels: Optional[int] = None):
        super().__init__()
        chans = [c.base * m for m in c.ch_mult]
        self.conv_in = Conv(in_channels or c.in_channels, chans[0], kt=c.kt)
        stages = []
        cur = chans[0]
        for i, ch in enumerate(chans):
            blocks = []
            for _ in range(c.num_res_blocks):
                blocks.append(ResBlock(cur, ch, c.kt))
                cur = ch
            if i < len(chans) - 1:
                blocks.append(Down(cur, bool(c.temporal_down[i]) and c.kt > 1, c.kt))
            stages.append(nn.Sequential(*blocks))
        self.stages = nn.ModuleList(stages)
        mid = [ResBlock(cur, cur, c.kt)] + ([SpatialAttention(cur)] if c.mid_attention else []) + [ResBlock(cur, cur, c.kt)]
        self.mid = nn.Sequential(*mid)
        self.norm_out = _norm(cur)
        self.conv_out = Conv(cur, (2 if c.double_z else 1) * c.z_channels, kt=c.kt)

    def forward(self, x, inject: Optional[List[Optional[torch.Tensor]]] = None):
        h = self.conv_in(x)
        for i, st in enumerate(self.stages):
            h = st(h)
            if inject is not None and i < len(inject) and inject[i] is not None:
                h = h + inject[i]
        return self.conv_out(F.silu(self.norm_out(self.mid(h))))


class Decoder(nn.Module):
    def __init__(self, c: KLVAEConfig, out_channels: Optional[int] = None):
        super().__init__()
        chans = [c.base * m for m in c.ch_mult][::-1]
        cur = chans[0]
        self.conv_in = Conv(c.z_channels, cur, kt=c.kt)
        mid = [ResBlock(cur, cur, c.kt)] + ([SpatialAttention(cur)] if c.mid_attention else []) + [ResBlock(cur, cur, c.kt)]
        self.mid = nn.Sequential(*mid)
        stages = []
        tdown = list(c.temporal_down)[::-1]
        for i, ch in enumerate(chans):
            blocks = []
            for _ in range(c.num_res_blocks + 1):
                blocks.append(ResBlock(cur, ch, c.kt))
                cur = ch
            if i < len(chans) - 1:
                blocks.append(Up(cur, bool(tdown[i]) and c.kt > 1, c.kt))
            stages.append(nn.Sequential(*blocks))
        self.stages = nn.ModuleList(stages)
        self.norm_out = _norm(cur)
        self.conv_out = Conv(cur, out_channels or c.out_channels, kt=c.kt)

    def forward(self, z):
        h = self.mid(self.conv_in(z))
        for st in self.stages:
            h = st(h)
        return self.conv_out(F.silu(self.norm_out(h)))


# ------------------------------------------------------------------------------------------------- assemblies
def _blend(a: torch.Tensor, b: torch.Tensor, dim: int, extent: int) -> torch.Tensor:
    """Cross-fades the last ``extent`` entries of ``a`` into the first ``extent`` of ``b`` along ``dim`` (returns b)."""
    extent = min(extent, a.shape[dim], b.shape[dim])
    if extent <= 0:
        return b
    w = torch.linspace(0, 1, extent + 2, device=b.device, dtype=b.dtype)[1:-1]
    shape = [1] * b.dim()
    shape[dim] = extent
    w = w.reshape(shape)
    head = a.narrow(dim, a.shape[dim] - extent, extent) * (1 - w) + b.narrow(dim, 0, extent) * w
    return torch.cat([head, b.narrow(dim, extent, b.shape[dim] - extent)], dim)


class CausalVAE3D(nn.Module):
    """Video (or, with ``kt = 1``, image) KL autoencoder; see the module docstring for the families it stands for."""

    def __init__(self, c: Optional[KLVAEConfig] = None, tile_sample_min: int = 256, tile_overlap: float = 0.25,
                 tile_frames: Optional[int] = None):
        super().__init__()
        self.c = c or KLVAEConfig.hunyuan_video()
        self.encoder, self.decoder = Encoder(self.c), Decoder(self.c)
        self.quant_conv = Conv(2 * self.c.z_channels, 2 * self.c.z_channels, k=1, kt=1)
        self.post_quant_conv = Conv(self.c.z_channels, self.c.z_channels, k=1, kt=1)
        self.use_tiling = False
        self.tile_sample_min, self.tile_overlap, self.tile_frames = tile_sample_min, tile_overlap, tile_frames

    def enable_tiling(self, on: bool = True):
        self.use_tiling = on

    def compression(self) -> Tuple[int, int, int]:
        return self.c.time_compression, self.c.spatial_compression, self.c.spatial_compression

    # ------------------------------------------------------------------ plain paths
    def _moments(self, x):
        return self.quant_conv(self.encoder(x))

    def _decode(self, z):
        return self.decoder(self.post_quant_conv(z))

    def _as_video(self, x):
        return (x[:, :, None], True) if x.dim() == 4 else (x, False)

    # ------------------------------------------------------------------ tiling
    def _tiles(self, x, fn, tile: int, scale: float):
        """Runs ``fn`` over overlapping H x W tiles and stitches with linear cross-fades.  ``scale`` = output / input
        size ratio of ``fn`` (1 / 8 for the encoder, 8 for the decoder)."""
        stride = max(1, int(tile * (1 - self.tile_overlap)))
        blend = int(round(tile * self.tile_overlap * scale))
        keep = int(round(stride * scale))
        rows = []
        for i in range(0, x.shape[3], stride):
            rows.append([fn(x[:, :, :, i:i + tile, j:j + tile]) for j in range(0, x.shape[4], stride)])
        out_rows = []
        for i, row in enumerate(rows):
            line = []
            for j, t in enumerate(row):
                if i > 0:
                    t = _blend(rows[i - 1][j], t, 3, blend)
                if j > 0:
                    t = _blend(row[j - 1], t, 4, blend)
                line.append(t[:, :, :, :keep, :keep])
            out_rows.append(torch.cat(line, 4))
        return torch.cat(out_rows, 3)

    def _time_chunks(self, x, fn, frames: Optional[int], latent: bool):
        """Temporal tiling.  Chunk 0 starts with the lone first frame; every later chunk is given the last frame (pixel
        or latent) of its predecessor as its own "first frame" and the output that frame produces is dropped, so
        each chunk is a valid 1 + k * compression clip and the pieces line up."""
        tc = self.c.time_compression
        if frames is None or x.shape[2] <= frames:
            return fn(x)
        step = max(1, frames) if latent else max(tc, (frames - 1) // tc * tc)
        outs, start = [fn(x[:, :, : 1 + step])], 1 + step
        while start < x.shape[2]:
            outs.append(fn(x[:, :, start - 1:start + step])[:, :, 1:])
            start += step
        return torch.cat(outs, 2)

    # ------------------------------------------------------------------ public
    def encode_moments(self, x):
        x, _ = self._as_video(x)
        s = self.c.spatial_compression
        fn = self._moments
        if self.use_tiling and max(x.shape[3], x.shape[4]) > self.tile_sample_min:
            inner = fn
            fn = lambda v: self._tiles(v, inner, self.tile_sample_min, 1.0 / s)      # noqa: E731
        return self._time_chunks(x, fn, self.tile_frames if self.use_tiling else None, latent=False)

    def encode(self, x, sample: bool = False, generator=None):
        was_image = x.dim() == 4
        post = DiagonalGaussian(self.encode_moments(x))
        z = post.sample(generator) if sample else post.mode()
        z = self.c.scale_factor * (z - self.c.shift_factor)
        return z[:, :, 0] if was_image else z

    def decode(self, z):
        z, was_image = self._as_video(z)
        z = z / self.c.scale_factor + self.c.shift_factor
        s = self.c.spatial_compression
        fn = self._decode
        tile = self.tile_sample_min // s
        if self.use_tiling and max(z.shape[3], z.shape[4]) > tile:
            inner = fn
            fn = lambda v: self._tiles(v, inner, tile, float(s))                      # noqa: E731
        lat_frames = None
        if self.use_tiling and self.tile_frames:
            lat_frames = max(1, (self.tile_frames - 1) // self.c.time_compression)
        out = self._time_chunks(z, fn, lat_frames, latent=True)
        return out[:, :, 0] if was_image else out

    def forward(self, x, sample_posterior: bool = True, generator=None):
        x5, was_image = self._as_video(x)
        post = DiagonalGaussian(self.encode_moments(x5))
        z = post.sample(generator) if sample_posterior else post.mode()
        rec = self._decode(z)
        return (rec[:, :, 0] if was_image else rec), post


class AutoencoderKL2D(CausalVAE3D):
    """Image VAE: a ``CausalVAE3D`` with temporal kernel 1 (every convolution is 2-D in effect)."""

    def __init__(self, c: Optional[KLVAEConfig] = None, **kw):
        c = c or KLVAEConfig.flux()
        if c.kt != 1:
            raise ValueError("AutoencoderKL2D needs kt = 1")
        super().__init__(c, **kw)


# ------------------------------------------------------------------------------------------------- wavelets
_H = torch.tensor([[1.0, 1.0], [1.0, -1.0]]) / math.sqrt(2.0)


def haar(x: torch.Tensor, dims: Sequence[int]) -> torch.Tensor:
    """Orthonormal Haar analysis along ``dims`` (each of even length) of ``[B, C, T, H, W]``; the 2^len(dims) bands are
    stacked on the channel axis, low-pass band first."""
    B, C = x.shape[:2]
    bands = [x]
    for d in dims:
        nxt = []
        for b in bands:
            even, odd = b.index_select(d, torch.arange(0, b.shape[d], 2, device=b.device)), \
                b.index_select(d, torch.arange(1, b.shape[d], 2, device=b.device))
            nxt.append((even + odd) / math.sqrt(2.0))
            nxt.append((even - odd) / math.sqrt(2.0))
        # keep "all low" first: order bands so that band k's bit i says high-pass along dims[i]
        bands = nxt[0::2] + nxt[1::2]
    return torch.cat(bands, 1)


def inverse_haar(w: torch.Tensor, dims: Sequence[int]) -> torch.Tensor:
    n = 2 ** len(dims)
    C = w.shape[1] // n
    bands = list(w.split(C, 1))
    for d in reversed(list(dims)):
        half = len(bands) // 2
        lows, highs = bands[:half], bands[half:]
        nxt = []
        for lo, hi in zip(lows, highs):
            even, odd = (lo + hi) / math.sqrt(2.0), (lo - hi) / math.sqrt(2.0)
            shape = list(even.shape)
            shape[d] *= 2
            nxt.append(torch.stack([even, odd], d + 1).reshape(shape))
        bands = nxt
    return bands[0]


def _causal_even(x):
    """Front-pads the time axis with a copy of the first frame when T is odd (1 + 2m -> 2 + 2m)."""
    return torch.cat([x[:, :, :1], x], 2) if x.shape[2] % 2 else x


class WFVAE(nn.Module):
    """Wavelet-flow VAE: compression 4 x 8 x 8.

    encoder:  W1 = Haar3D(video)                      -> conv_in, stage 0                     (T/2, H/2, W/2)
              W2 = Haar2D(low band of W1)  -> inflow  -> added after the spatial down stage    (T/2, H/4, W/4)
              W3 = Haar3D(low band of W2)  -> inflow  -> added after the 3-D down stage        (T/4, H/8, W/8)
    decoder:  mirrors it; each level predicts its wavelet coefficients, the inverse transform of level k + 1 is added to
              the low band of level k ("energy flow"), and the video is the inverse Haar3D of the level-1 prediction.
    """

    def __init__(self, base: int = 128, z_channels: int = 8, in_channels: int = 3, num_res_blocks: int = 2, energy_flow: int = 64,
                 scale_factor: float = 1.0, shift_factor: float = 0.0, mid_attention: bool = True):
        super().__init__()
        c = KLVAEConfig(in_channels=8 * in_channels, out_channels=8 * in_channels, base=base, ch_mult=(1, 2, 4),
                        num_res_blocks=num_res_blocks, z_channels=z_channels, temporal_down=(False, True), kt=3,
                        mid_attention=mid_attention, scale_factor=scale_factor, shift_factor=shift_factor)
        self.c, self.in_channels = c, in_channels
        self.encoder = Encoder(c)
        self.in_flow2 = nn.Sequential(Conv(4 * in_channels, energy_flow, kt=1), ResBlock(energy_flow, base, 1))
        self.in_flow3 = nn.Sequential(Conv(8 * in_channels, energy_flow), ResBlock(energy_flow, 2 * base, 3))
        # decoder trunk, split by stage so the wavelet predictions can leave it
        self.decoder = Decoder(c)
        self.out_flow3 = nn.Sequential(ResBlock(4 * base, energy_flow, 3), Conv(energy_flow, 8 * in_channels))
        self.out_flow2 = nn.Sequential(ResBlock(2 * base, energy_flow, 1), Conv(energy_flow, 4 * in_channels, kt=1))

    def compression(self):
        return 4, 8, 8

    def _analysis(self, x):
        w1 = haar(_causal_even(x), (2, 3, 4))
        low1 = w1[:, : self.in_channels]
        w2 = haar(low1, (3, 4))
        low2 = w2[:, : self.in_channels]
        w3 = haar(_causal_even(low2), (2, 3, 4))
        return w1, w2, w3

    def encode_moments(self, x):
        w1, w2, w3 = self._analysis(x)
        return self.encoder(w1, inject=[self.in_flow2(w2), self.in_flow3(w3)])

    def encode(self, x, sample: bool = False, generator=None):
        post = DiagonalGaussian(self.encode_moments(x))
        z = post.sample(generator) if sample else post.mode()
        return self.c.scale_factor * (z - self.c.shift_factor)

    def _decode(self, z, frames: Optional[int] = None):
        d = self.decoder
        h = d.mid(d.conv_in(z))
        h = d.stages[0][:-1](h)                                  # T/4, H/8
        w3 = self.out_flow3(h)
        h = d.stages[0][-1](h)                                   # up 3-D -> T/2, H/4
        h = d.stages[1][:-1](h)
        w2 = self.out_flow2(h)
        low2 = inverse_haar(w3, (2, 3, 4))
        low2 = low2[:, :, low2.shape[2] - w2.shape[2]:]          # drop the causal pad frame
        w2 = torch.cat([w2[:, : self.in_channels] + low2, w2[:, self.in_channels:]], 1)
        h = d.stages[1][-1](h)                                   # up 2-D -> T/2, H/2
        h = d.stages[2](h)
        w1 = d.conv_out(F.silu(d.norm_out(h)))
        low1 = inverse_haar(w2, (3, 4))
        w1 = torch.cat([w1[:, : self.in_channels] + low1, w1[:, self.in_channels:]], 1)
        video = inverse_haar(w1, (2, 3, 4))
        return video[:, :, 1:] if frames is None or video.shape[2] > frames else video

    def decode(self, z):
        return self._decode(z / self.c.scale_factor + self.c.shift_factor)

    def forward(self, x, sample_posterior: bool = True, generator=None):
        post = DiagonalGaussian(self.encode_moments(x))
        z = post.sample(generator) if sample_posterior else post.mode()
        return self._decode(z, x.shape[2]), post

    def get_last_layer(self):
        return self.decoder.conv_out.conv.weight


# ------------------------------------------------------------------------------------------------- VQ tokenizer
class VectorQuantizer(nn.Module):
    def __init__(self, n_embed: int, dim: int):
        super().__init__()
        self.embedding = nn.Embedding(n_embed, dim)
        nn.init.uniform_(self.embedding.weight, -1.0 / n_embed, 1.0 / n_embed)

    def forward(self, z):
        """``z`` [B, D, H, W] -> (indices [B, H, W], quantised [B, D, H, W] with straight-through gradient, commit loss)."""
        B, D, H, W = z.shape
        flat = z.permute(0, 2, 3, 1).reshape(-1, D).float()
        e = self.embedding.weight.float()
        dist = flat.pow(2).sum(1, keepdim=True) - 2 * flat @ e.t() + e.pow(2).sum(1)
        idx = dist.argmin(1)
        q = self.embedding(idx).reshape(B, H, W, D).permute(0, 3, 1, 2).to(z.dtype)
        commit = F.mse_loss(q.detach(), z) * 0.25 + F.mse_loss(q, z.detach())
        return idx.reshape(B, H, W), z + (q - z).detach(), commit


class MOVQ(nn.Module):
    def __init__(self, z_channels: int = 4, in_channels: int = 3, base: int = 256, ch_mult: Sequence[int] = (1, 2, 2, 4),
                 num_res_blocks: int = 2, n_embed: int = 16384, embed_dim: int = 4, mid_attention: bool = True, **_):
        super().__init__()
        c = KLVAEConfig(in_channels=in_channels, out_channels=in_channels, base=base, ch_mult=tuple(ch_mult),
                        num_res_blocks=num_res_blocks, z_channels=z_channels, kt=1, mid_attention=mid_attention, double_z=False,
                        temporal_down=(False,) * (len(ch_mult) - 1))
        self.c = c
        self.encoder, self.decoder = Encoder(c), Decoder(c)
        self.quantize = VectorQuantizer(n_embed, embed_dim)
        self.quant_conv = nn.Conv2d(z_channels, embed_dim, 1)
        self.post_quant_conv = nn.Conv2d(embed_dim, z_channels, 1)

    def encode(self, x):
        """Image [B, 3, H, W] -> code indices [B, H/8, W/8] (what the autoregressive image-token models consume)."""
        h = self.quant_conv(self.encoder(x[:, :, None])[:, :, 0])
        return self.quantize(h)[0]

    def decode_codes(self, idx):
        q = self.quantize.embedding(idx).permute(0, 3, 1, 2)
        return self.decoder(self.post_quant_conv(q)[:, :, None])[:, :, 0]

    def forward(self, x):
        h = self.quant_conv(self.encoder(x[:, :, None])[:, :, 0])
        idx, q, commit = self.quantize(h)
        return self.decoder(self.post_quant_conv(q)[:, :, None])[:, :, 0], idx, commit
