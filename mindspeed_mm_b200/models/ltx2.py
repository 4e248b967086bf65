"""LTX-2 style joint audio-video diffusion transformer.

Two token streams (video latents, audio latents) run through the same stack of blocks.  In every block each stream
does: adaLN-modulated self-attention with rotary positions -> cross-attention to its text context; then the two
streams exchange information through a pair of cross-attentions (audio -> video and video -> audio) whose inputs are
modulated by their own timestep tables; then an adaLN-modulated feed-forward.  Timesteps are per token, so clean
conditioning frames and noisy frames can share a sequence.  Either stream may be absent.

Reference: the training wrapper and block forward of mindspeed_mm/fsdp/models/ltx2/ltx2_fsdp2/{modeling_ltx2.py:44,
modified.py:8-170} (the transformer itself comes from the external ``ltx_core`` package there); ``ltx2_3`` uses the same
block with a different configuration.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .qwen2_5_vl import Linear
from .registry import model_register
from .wan import sinusoidal_embedding


@dataclass
class LTX2Config:
    num_layers: int = 48
    dim: int = 4096                    # video stream width
    audio_dim: int = 2048
    num_heads: int = 32
    audio_heads: int = 32
    in_channels: int = 128             # video latent channels per token (already patchified)
    audio_in_channels: int = 128
    caption_dim: int = 3840
    ff_mult: int = 4
    freq_dim: int = 256
    rope_theta: float = 10000.0
    rope_axes: Tuple[int, int, int] = (20, 2048, 2048)     # largest position per video axis (t, h, w) used to normalise
    audio_rope_max: int = 20
    norm_eps: float = 1e-6
    video: bool = True
    audio: bool = True

    @staticmethod
    def tiny(**kw):
        d = dict(num_layers=2, dim=64, audio_dim=32, num_heads=4, audio_heads=2, in_channels=8, audio_in_channels=6, caption_dim=24,
                 freq_dim=16)
        d.update(kw)
        return LTX2Config(**d)


def rms(x, eps):
    return x * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps).to(x.dtype)


def fractional_rope(positions: torch.Tensor, head_dim: int, theta: float, maxima) -> Tuple[torch.Tensor, torch.Tensor]:
    """``positions`` [B, A, S] (A axes, real-valued) -> cos / sin [B, S, head_dim / 2].  The rotary pairs are dealt out to
    the axes in equal shares.  Every axis is mapped to [-1, 1] by its maximum and multiplied by a geometric ladder of
    frequencies ``theta ** [0 .. 1] * pi / 2``, so the angles depend on the relative, not the absolute, position."""
    B, A, S = positions.shape
    half = head_dim // 2
    per = half // A
    angles = []
    for a in range(A):
        n = per if a < A - 1 else half - per * (A - 1)
        freqs = theta ** torch.linspace(0.0, 1.0, n, device=positions.device) * (math.pi / 2)
        frac = positions[:, a].float() / float(maxima[a])
        angles.append((2.0 * frac - 1.0)[:, :, None] * freqs)
    ang = torch.cat(angles, -1)
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    """x [B, S, N, D] with interleaved pairs; cos / sin [B, S, D / 2]."""
    x1, x2 = x.float()[..., 0::2], x.float()[..., 1::2]
    c, s = cos[:, :, None], sin[:, :, None]
    return torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], -1).flatten(-2).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, q_dim, kv_dim, heads, eps):
        super().__init__()
        self.h, self.hd = heads, q_dim // heads
        self.to_q, self.to_k, self.to_v = Linear(q_dim, q_dim), Linear(kv_dim, q_dim), Linear(kv_dim, q_dim)
        self.to_out = Linear(q_dim, q_dim)
        self.q_norm = nn.Parameter(torch.ones(q_dim))
        self.k_norm = nn.Parameter(torch.ones(q_dim))
        self.eps = eps

    def forward(self, x, context=None, mask=None, pe=None, k_pe=None):
        ctx = x if context is None else context
        B, S, _ = x.shape
        L = ctx.shape[1]
        q = (rms(self.to_q(x), self.eps) * self.q_norm).view(B, S, self.h, self.hd)
        k = (rms(self.to_k(ctx), self.eps) * self.k_norm).view(B, L, self.h, self.hd)
        v = self.to_v(ctx).view(B, L, self.h, self.hd)
        if pe is not None:
            q = apply_rope(q, *pe)
            k = apply_rope(k, *(k_pe if k_pe is not None else pe))
        if mask is None:
            o = ops.attention_dense(q, k, v)
        else:
            bias = torch.zeros(B, 1, 1, L, dtype=q.dtype, device=q.device).masked_fill(~mask.bool()[:, None, None], float("-inf"))
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=bias).transpose(1, 2)
        return self.to_out(o.reshape(B, S, self.h * self.hd))


class FeedForward(nn.Module):
    def __init__(self, dim, mult):
        super().__init__()
        self.up, self.down = Linear(dim, mult * dim), Linear(mult * dim, dim)

    def forward(self, x):
        return self.down(ops.gelu_tanh(self.up(x)))


class TimeEmbed(nn.Module):
    """Per-token timestep -> (modulation vector of ``n * dim``, embedded timestep of ``dim``)."""

    def __init__(self, dim, freq_dim, n):
        super().__init__()
        self.freq_dim = freq_dim
        self.l1, self.l2 = Linear(freq_dim, dim), Linear(dim, dim)
        self.proj = Linear(dim, n * dim)

    def forward(self, t):
        B, S = t.shape
        uniq, inv = torch.unique(t.reshape(-1), return_inverse=True)
        e = self.l2(F.silu(self.l1(sinusoidal_embedding(uniq, self.freq_dim).to(self.l1.weight.dtype))))
        return self.proj(F.silu(e))[inv].view(B, S, -1), e[inv].view(B, S, -1)


class AVBlock(nn.Module):
    def __init__(self, c: LTX2Config):
        super().__init__()
        self.eps = c.norm_eps
        D, A = c.dim, c.audio_dim
        if c.video:
            self.attn1, self.attn2 = Attention(D, D, c.num_heads, c.norm_eps), Attention(D, D, c.num_heads, c.norm_eps)
            self.ff = FeedForward(D, c.ff_mult)
            self.scale_shift_table = nn.Parameter(torch.randn(6, D) / D ** 0.5)
        if c.audio:
            self.audio_attn1, self.audio_attn2 = Attention(A, A, c.audio_heads, c.norm_eps), Attention(A, A, c.audio_heads, c.norm_eps)
            self.audio_ff = FeedForward(A, c.ff_mult)
            self.audio_scale_shift_table = nn.Parameter(torch.randn(6, A) / A ** 0.5)
        if c.video and c.audio:
            self.audio_to_video_attn = Attention(D, A, c.num_heads, c.norm_eps)
            self.video_to_audio_attn = Attention(A, D, c.audio_heads, c.norm_eps)
            self.scale_shift_table_a2v_ca_video = nn.Parameter(torch.randn(5, D) / D ** 0.5)
            self.scale_shift_table_a2v_ca_audio = nn.Parameter(torch.randn(5, A) / A ** 0.5)

    @staticmethod
    def _ada(table, temb, sl):
        """table [n, D] + temb [B, S, n * D] -> the requested rows as [B, S, D] tensors."""
        n, D = table.shape
        vals = table.to(temb.dtype)[None, None] + temb.view(temb.shape[0], temb.shape[1], n, D)
        return vals[:, :, sl].unbind(2)

    def forward(self, vx, ax, v: Optional[dict], a: Optional[dict]):
        eps = self.eps
        if vx is not None:
            sh, sc, g = self._ada(self.scale_shift_table, v["temb"], slice(0, 3))
            vx = vx + self.attn1(rms(vx, eps) * (1 + sc) + sh, pe=v["pe"]) * g
            vx = vx + self.attn2(rms(vx, eps), context=v["context"], mask=v.get("context_mask"))
        if ax is not None:
            sh, sc, g = self._ada(self.audio_scale_shift_table, a["temb"], slice(0, 3))
            ax = ax + self.audio_attn1(rms(ax, eps) * (1 + sc) + sh, pe=a["pe"]) * g
            ax = ax + self.audio_attn2(rms(ax, eps), context=a["context"], mask=a.get("context_mask"))
        if vx is not None and ax is not None:
            vn, an = rms(vx, eps), rms(ax, eps)
            a_sc_a2v, a_sh_a2v, a_sc_v2a, a_sh_v2a, g_v2a = self._ada(self.scale_shift_table_a2v_ca_audio, a["cross_temb"], slice(0, 5))
            v_sc_a2v, v_sh_a2v, v_sc_v2a, v_sh_v2a, g_a2v = self._ada(self.scale_shift_table_a2v_ca_video, v["cross_temb"], slice(0, 5))
            vx = vx + self.audio_to_video_attn(vn * (1 + v_sc_a2v) + v_sh_a2v, context=an * (1 + a_sc_a2v) + a_sh_a2v,
                                               pe=v["cross_pe"], k_pe=a["cross_pe_k"]) * g_a2v
            ax = ax + self.video_to_audio_attn(an * (1 + a_sc_v2a) + a_sh_v2a, context=vn * (1 + v_sc_v2a) + v_sh_v2a,
                                               pe=a["cross_pe"], k_pe=v["cross_pe_k"]) * g_v2a
        if vx is not None:
            sh, sc, g = self._ada(self.scale_shift_table, v["temb"], slice(3, 6))
            vx = vx + self.ff(rms(vx, eps) * (1 + sc) + sh) * g
        if ax is not None:
            sh, sc, g = self._ada(self.audio_scale_shift_table, a["temb"], slice(3, 6))
            ax = ax + self.audio_ff(rms(ax, eps) * (1 + sc) + sh) * g
        return vx, ax


class _StreamIO(nn.Module):
    """Input projection, timestep embedders, caption projection and the modulated output head of one stream."""

    def __init__(self, in_ch, dim, caption_dim, freq_dim, cross: bool):
        super().__init__()
        self.patchify_proj = Linear(in_ch, dim)
        self.adaln = TimeEmbed(dim, freq_dim, 6)
        self.cross_adaln = TimeEmbed(dim, freq_dim, 5) if cross else None
        self.caption_1, self.caption_2 = Linear(caption_dim, dim), Linear(dim, dim)
        self.out_table = nn.Parameter(torch.randn(2, dim) / dim ** 0.5)
        self.proj_out = Linear(dim, in_ch)

    def forward(self, mode: str, *args):
        """One sharding unit, two entry points: ``("prepare", latent, timesteps, context)`` and ``("output", x, emb, eps)``."""
        return self.prepare(*args) if mode == "prepare" else self.output(*args)

    def prepare(self, latent, timesteps, context):
        x = self.patchify_proj(latent.to(self.patchify_proj.weight.dtype))
        temb, emb = self.adaln(timesteps)
        d = dict(temb=temb, emb=emb, context=self.caption_2(ops.gelu_tanh(self.caption_1(context.to(x.dtype)))))
        if self.cross_adaln is not None:
            d["cross_temb"] = self.cross_adaln(timesteps)[0]
        return x, d

    def output(self, x, emb, eps):
        sh, sc = (self.out_table.to(x.dtype)[None, None] + emb[:, :, None]).unbind(2)
        return self.proj_out(rms(x, eps) * (1 + sc) + sh)


@model_register.register("ltx2")
class LTX2Model(nn.Module):
    """``forward(video_latent [B, Sv, Cv], video_timesteps [B, Sv], video_positions [B, 3, Sv], context [B, L, Cc],
    video_target_velocity, audio_latent / audio_timesteps / audio_positions [B, 1, Sa] / audio_target_velocity, context_mask,
    loss_mask)`` -> dict(loss, video_pred, audio_pred); without targets only the predictions are filled."""
    config_class = LTX2Config

    def __init__(self, config: Optional[LTX2Config] = None):
        super().__init__()
        self.config = c = config or LTX2Config.tiny()
        both = c.video and c.audio
        self.video_io = _StreamIO(c.in_channels, c.dim, c.caption_dim, c.freq_dim, both) if c.video else None
        self.audio_io = _StreamIO(c.audio_in_channels, c.audio_dim, c.caption_dim, c.freq_dim, both) if c.audio else None
        self.transformer_blocks = nn.ModuleList(AVBlock(c) for _ in range(c.num_layers))

    def fsdp_units(self):
        u = [("video_io", self.video_io)] if self.video_io is not None else []
        u += [("audio_io", self.audio_io)] if self.audio_io is not None else []
        return u + [(f"transformer_blocks.{i}", b) for i, b in enumerate(self.transformer_blocks)]

    def forward(self, video_latent=None, video_timesteps=None, video_positions=None, context=None, video_target_velocity=None,
                context_mask=None, loss_mask=None, audio_latent=None, audio_timesteps=None, audio_positions=None,
                audio_target_velocity=None, audio_context=None, audio_context_mask=None, run=None, **_):
        if isinstance(video_latent, dict):
            # engine convention ``model(batch, run=...)``: unpack the batch and hand back the scalar loss
            return self.forward(**video_latent, run=run)["loss"]
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        vx = ax = v = a = None
        hd_v, hd_a = c.dim // c.num_heads, c.audio_dim // c.audio_heads
        if video_latent is not None and self.video_io is not None:
            vx, v = run(self.video_io, "prepare", video_latent, video_timesteps, context)
            v["context_mask"] = context_mask
            v["pe"] = fractional_rope(video_positions, c.dim // c.num_heads, c.rope_theta, c.rope_axes)
            # the audio <-> video attentions share only the time axis; as keys of the audio queries the video tokens
            # need a table of the audio head width
            t_axis = video_positions[:, :1]
            v["cross_pe"] = fractional_rope(t_axis, hd_v, c.rope_theta, c.rope_axes[:1])
            v["cross_pe_k"] = fractional_rope(t_axis, hd_a, c.rope_theta, c.rope_axes[:1])
        if audio_latent is not None and self.audio_io is not None:
            if audio_timesteps is None or audio_positions is None:
                raise ValueError("audio_timesteps and audio_positions are required with audio_latent")
            ax, a = run(self.audio_io, "prepare", audio_latent, audio_timesteps, audio_context if audio_context is not None else context)
            a["context_mask"] = audio_context_mask if audio_context_mask is not None else context_mask
            a["pe"] = fractional_rope(audio_positions, c.audio_dim // c.audio_heads, c.rope_theta, (c.audio_rope_max,))
            a["cross_pe"] = fractional_rope(audio_positions[:, :1], hd_a, c.rope_theta, c.rope_axes[:1])
            a["cross_pe_k"] = fractional_rope(audio_positions[:, :1], hd_v, c.rope_theta, c.rope_axes[:1])
        for blk in self.transformer_blocks:
            vx, ax = run(blk, vx, ax, v, a)
        out = dict(loss=None, video_pred=None, audio_pred=None)
        losses = []
        if vx is not None:
            out["video_pred"] = run(self.video_io, "output", vx, v["emb"], c.norm_eps)
            if video_target_velocity is not None:
                err = (out["video_pred"].float() - video_target_velocity.float()) ** 2
                if loss_mask is not None:
                    m = loss_mask.to(err.dtype)[..., None]
                    losses.append((err * m).sum() / (m.sum().clamp(min=1) * err.shape[-1]))
                else:
                    losses.append(err.mean())
        if ax is not None:
            out["audio_pred"] = run(self.audio_io, "output", ax, a["emb"], c.norm_eps)
            if audio_target_velocity is not None:
                losses.append(((out["audio_pred"].float() - audio_target_velocity.float()) ** 2).mean())
        if losses:
            out["loss"] = sum(losses)
        return out


@model_register.register("ltx2_3")
class LTX23Model(LTX2Model):
    """Same block; the 2.3 checkpoints differ in depth / widths only, which come from the configuration."""
