"""Wan2.1 / 2.2 video DiT (t2v, i2v) with adaLN-zero modulation, QK-RMSNorm, 3-D RoPE and text cross-attention.

Architecture facts reproduced from the reference's WanDiT (mindspeed_mm/models/predictor/dits/wan_dit.py:33-1163;
dims in examples/wan2.1/14b/t2v/pretrain_model.json):
  * time path: sinusoid(freq_dim) -> Linear-SiLU-Linear = ``times`` [B,H]; SiLU-Linear -> [B,6,H] modulation
  * block: x += gate_msa * SelfAttn(LN(x)(1+scale_msa)+shift_msa); x += CrossAttn(LN_affine(x), text);
           x += gate_mlp * FFN(LN(x)(1+scale_mlp)+shift_mlp);  modulation = learned [1,6,H] + time projection
  * q and k pass an RMSNorm over the FULL hidden size before the head split; 3-D RoPE rotates interleaved pairs
    with the head dim split (44, 42, 42) over (frame, height, width) for D = 128
  * head: LN(x)(1+e1)+e0 with e = learned [1,2,H] + times, then Linear to patch pixels, then unpatchify
  * i2v adds CLIP image tokens: extra k_img / v_img projections whose attention output is summed with the text one
Sequence parallelism: tokens are split over the Ulysses group right after patchify (RoPE tables split the same
way) and gathered before the head; cross-attention needs no communication (wan_dit.py:412-471,988-990).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel.cp.split import cal_split_sizes, gather_forward_split_backward, split_forward_gather_backward
from ..parallel.cp.ulysses import ulysses_attention
from ..parallel.state import get_parallel_state
from .qwen2_5_vl import Linear
from .registry import model_register


import os as _os
# "fused" (default): Ulysses collectives inside the projection GEMMs over peer memory; "nccl": all-to-all collectives
_ULYSSES_PATH = _os.environ.get("MM_B200_ULYSSES", "fused")


@dataclass
class WanConfig:
    model_type: str = "t2v"
    patch_size: Sequence[int] = (1, 2, 2)
    text_len: int = 512
    in_dim: int = 16
    hidden_size: int = 5120
    ffn_dim: int = 13824
    freq_dim: int = 256
    text_dim: int = 4096
    img_dim: int = 1280
    out_dim: int = 16
    num_heads: int = 40
    num_layers: int = 40
    qk_norm: bool = True
    cross_attn_norm: bool = True
    eps: float = 1e-6
    rope_theta: float = 10000.0
    init_std: float = 0.02

    @staticmethod
    def wan2_1_14b():
        return WanConfig()

    @staticmethod
    def wan2_1_1_3b():
        return WanConfig(hidden_size=1536, ffn_dim=8960, num_heads=12, num_layers=30)

    @staticmethod
    def tiny():
        return WanConfig(hidden_size=128, ffn_dim=256, num_heads=4, num_layers=2, text_dim=64, text_len=16, freq_dim=32)

    @staticmethod
    def from_mm_json(pred: dict) -> "WanConfig":
        keys = WanConfig.__dataclass_fields__.keys()
        return WanConfig(**{k: v for k, v in pred.items() if k in keys})


def sinusoidal_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    """fp64 sinusoid, [cos | sin] halves (wan_dit.py:231-242)."""
    half = dim // 2
    pos = t.to(torch.float64).reshape(-1, 1)
    freqs = torch.pow(10000.0, -torch.arange(half, dtype=torch.float64, device=t.device) / half)
    ang = pos * freqs
    return torch.cat([ang.cos(), ang.sin()], dim=1).float()


class FullRMSNorm(nn.Module):
    """RMSNorm over the whole hidden vector (all heads together)."""

    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)


class AffineLayerNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))
        self.eps = eps

    def forward(self, x):
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class WanSelfAttention(nn.Module):
    def __init__(self, c: WanConfig):
        super().__init__()
        self.nh, self.hd = c.num_heads, c.hidden_size // c.num_heads
        self.qkv = Linear(c.hidden_size, 3 * c.hidden_size)          # fused proj_q | proj_k | proj_v
        self.proj_out = Linear(c.hidden_size, c.hidden_size)
        self.q_norm = FullRMSNorm(c.hidden_size, c.eps) if c.qk_norm else nn.Identity()
        self.k_norm = FullRMSNorm(c.hidden_size, c.eps) if c.qk_norm else nn.Identity()

    def _fused_group(self, x, seq_sizes, rope_full):
        """The Ulysses group when the fused peer-memory path applies: native tier on CUDA, one sample, equal sequence
        slices, whole-row q/k norm present, head block per rank a multiple of 64 channels."""
        if rope_full is None or seq_sizes is not None or x.shape[0] != 1 or not isinstance(self.q_norm, FullRMSNorm):
            return None
        ps = get_parallel_state()
        if not ps.enabled("ulysses") or _ULYSSES_PATH == "nccl":
            return None
        from ..comm import fused
        if not fused.fused_supported(x):
            return None
        world = ps.size("ulysses")
        H = x.shape[-1]
        if self.nh % world or (H // world) % 64 or world > 8:
            return None
        return ps.get_ulysses_group()

    def _forward_fused(self, x, rope_full, group):
        """Self-attention under Ulysses with every collective inside a GEMM (``comm/fused.py``): the QKV projection stores
        each head block into its owner (and emits the row sums of squares the whole-row q/k norm needs), the owner
        normalises + rotates its heads and runs attention over the full sequence, the output projection fetches the heads
        back inside its GEMM; the backward passes mirror this."""
        import torch.distributed as dist
        from ..comm import fused
        S_local, H = x.shape[1], x.shape[2]
        world = dist.get_world_size(group)
        dev = x.device
        qkv = fused.shared(fused.UlyssesQKVProjection, group, dev, S_local, 3 * H, 3, True)
        raw, stats = qkv(x[0], self.qkv.weight, self.qkv.bias)
        nr = fused.shared(fused.UlyssesQKNormRope, group, dev, S_local * world, H // world, self.hd, H, self.q_norm.eps)
        q, k, v = nr(raw, stats, self.q_norm.weight, self.k_norm.weight, rope_full[0], rope_full[1])
        o = ops.attention_dense(q[None], k[None], v[None])[0]                   # [S_full, heads / world, D]
        out = fused.shared(fused.UlyssesOutProjection, group, dev, S_local, H)
        return out(o.reshape(S_local * world, H // world), self.proj_out.weight, self.proj_out.bias)[None]

    def forward(self, x, rope, seq_sizes, rope_full=None):
        B, S, H = x.shape
        group = self._fused_group(x, seq_sizes, rope_full)
        if group is not None:
            return self._forward_fused(x, rope_full, group)
        q, k, v = self.qkv(x).split(H, dim=-1)
        q, k = self.q_norm(q), self.k_norm(k)
        cos, sin = rope
        q = ops.rope_interleaved(q.reshape(B * S, self.nh, self.hd), cos, sin).view(B, S, self.nh, self.hd)
        k = ops.rope_interleaved(k.reshape(B * S, self.nh, self.hd), cos, sin).view(B, S, self.nh, self.hd)
        v = v.reshape(B, S, self.nh, self.hd)
        ps = get_parallel_state()
        o = ulysses_attention(lambda a, b, c: ops.attention_dense(a, b, c), q, k, v,
                              ps.get_ulysses_group() if ps.enabled("ulysses") else None, seq_sizes=seq_sizes)
        return self.proj_out(o.reshape(B, S, H))


class WanCrossAttention(nn.Module):
    def __init__(self, c: WanConfig):
        super().__init__()
        self.nh, self.hd = c.num_heads, c.hidden_size // c.num_heads
        self.i2v = c.model_type in ("i2v", "flf2v")
        self.proj_q = Linear(c.hidden_size, c.hidden_size)
        self.kv = Linear(c.hidden_size, 2 * c.hidden_size)           # fused proj_k | proj_v (text)
        self.proj_out = Linear(c.hidden_size, c.hidden_size)
        self.q_norm = FullRMSNorm(c.hidden_size, c.eps) if c.qk_norm else nn.Identity()
        self.k_norm = FullRMSNorm(c.hidden_size, c.eps) if c.qk_norm else nn.Identity()
        if self.i2v:
            self.kv_img = Linear(c.hidden_size, 2 * c.hidden_size)
            self.k_norm_img = FullRMSNorm(c.hidden_size, c.eps) if c.qk_norm else nn.Identity()

    def forward(self, x, ctx, n_img: int = 0):
        B, S, H = x.shape
        q = self.q_norm(self.proj_q(x)).view(B, S, self.nh, self.hd)
        txt = ctx[:, n_img:]
        k, v = self.kv(txt).split(H, dim=-1)
        k = self.k_norm(k)
        L = txt.shape[1]
        o = ops.attention_dense(q, k.reshape(B, L, self.nh, self.hd), v.reshape(B, L, self.nh, self.hd))
        if self.i2v and n_img:
            ki, vi = self.kv_img(ctx[:, :n_img]).split(H, dim=-1)
            ki = self.k_norm_img(ki)
            o = o + ops.attention_dense(q, ki.reshape(B, n_img, self.nh, self.hd), vi.reshape(B, n_img, self.nh, self.hd))
        return self.proj_out(o.reshape(B, S, H))


class WanBlock(nn.Module):
    def __init__(self, c: WanConfig):
        super().__init__()
        self.eps = c.eps
        self.modulation = nn.Parameter(torch.zeros(1, 6, c.hidden_size))
        self.self_attn = WanSelfAttention(c)
        self.norm3 = AffineLayerNorm(c.hidden_size, c.eps) if c.cross_attn_norm else nn.Identity()
        self.cross_attn = WanCrossAttention(c)
        self.ffn_0 = Linear(c.hidden_size, c.ffn_dim)
        self.ffn_2 = Linear(c.ffn_dim, c.hidden_size)

    def forward(self, x, time_emb, ctx, rope_cos, rope_sin, seq_sizes=None, n_img: int = 0, rope_full=None):
        e = (self.modulation.to(time_emb.dtype) + time_emb).chunk(6, dim=1)         # each [B,1,H]
        y = self.self_attn(ops.layer_norm_modulate(x, e[1], e[0], self.eps), (rope_cos, rope_sin), seq_sizes, rope_full)
        x = ops.gated_residual(x, y, e[2])
        x = x + self.cross_attn(self.norm3(x), ctx, n_img)
        y = self.ffn_2(ops.gelu_tanh(self.ffn_0(ops.layer_norm_modulate(x, e[4], e[3], self.eps))))
        return ops.gated_residual(x, y, e[5])


class WanEmbeddings(nn.Module):
    """Patch, text and time embeddings (the pipeline-first-stage tensors of the reference)."""

    def __init__(self, c: WanConfig):
        super().__init__()
        self.c = c
        p = c.patch_size
        self.patch_embedding = Linear(c.in_dim * p[0] * p[1] * p[2], c.hidden_size)
        self.text_embedding_1 = Linear(c.text_dim, c.hidden_size)
        self.text_embedding_2 = Linear(c.hidden_size, c.hidden_size)
        self.time_embedding_0 = Linear(c.freq_dim, c.hidden_size)
        self.time_embedding_2 = Linear(c.hidden_size, c.hidden_size)
        self.time_projection = Linear(c.hidden_size, 6 * c.hidden_size)
        if c.model_type in ("i2v", "flf2v"):
            self.img_emb_norm1 = AffineLayerNorm(c.img_dim, 1e-5)
            self.img_emb_fc1 = Linear(c.img_dim, c.img_dim)
            self.img_emb_fc2 = Linear(c.img_dim, c.hidden_size)
            self.img_emb_norm2 = AffineLayerNorm(c.hidden_size, 1e-5)

    def patchify(self, x):
        """[B, C, F, H, W] -> [B, f*h*w, C*pf*ph*pw] in Conv3d weight order (C, pf, ph, pw)."""
        B, C, Fr, Hh, Ww = x.shape
        pf, ph, pw = self.c.patch_size
        x = x.view(B, C, Fr // pf, pf, Hh // ph, ph, Ww // pw, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, (Fr // pf) * (Hh // ph) * (Ww // pw), C * pf * ph * pw), (Fr // pf, Hh // ph, Ww // pw)

    def forward(self, latents, timestep, prompt, clip_feature=None):
        dtype = self.patch_embedding.weight.dtype
        tokens, grid = self.patchify(latents.to(dtype))
        x = self.patch_embedding(tokens)
        te = sinusoidal_embedding(timestep, self.c.freq_dim).to(dtype)
        times = self.time_embedding_2(F.silu(self.time_embedding_0(te)))                      # [B, H]
        time_emb = self.time_projection(F.silu(times)).view(times.shape[0], 6, -1)            # [B, 6, H]
        ctx = self.text_embedding_2(ops.gelu_tanh(self.text_embedding_1(prompt.to(dtype))))
        n_img = 0
        if clip_feature is not None:
            img = self.img_emb_norm2(self.img_emb_fc2(ops.gelu(self.img_emb_fc1(self.img_emb_norm1(clip_feature.to(dtype))))))
            ctx = torch.cat([img, ctx], dim=1)
            n_img = img.shape[1]
        return x, times, time_emb, ctx, n_img


class WanHead(nn.Module):
    def __init__(self, c: WanConfig):
        super().__init__()
        self.c = c
        p = c.patch_size
        self.modulation = nn.Parameter(torch.zeros(1, 2, c.hidden_size))
        self.head = Linear(c.hidden_size, c.out_dim * p[0] * p[1] * p[2])

    def forward(self, x, times):
        e = (self.modulation.to(times.dtype) + times.unsqueeze(1)).chunk(2, dim=1)
        return self.head(ops.layer_norm_modulate(x, e[1], e[0], self.c.eps))

    def unpatchify(self, y, grid):
        B = y.shape[0]
        f, h, w = grid
        pf, ph, pw = self.c.patch_size
        y = y.view(B, f, h, w, pf, ph, pw, self.c.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return y.reshape(B, self.c.out_dim, f * pf, h * ph, w * pw)


@model_register.register("wandit")
class WanDiT(nn.Module):
    """``forward(latents [B,C,F,H,W], timestep [B], prompt [B,L,text_dim], clip_feature=None) -> [B,C,F,H,W]``."""
    config_class = WanConfig

    def __init__(self, config: WanConfig):
        super().__init__()
        self.config = config
        self.embeddings = WanEmbeddings(config)
        self.blocks = nn.ModuleList([WanBlock(config) for _ in range(config.num_layers)])
        self.head = WanHead(config)

    def fsdp_units(self):
        return [("embeddings", self.embeddings)] + [(f"blocks.{i}", b) for i, b in enumerate(self.blocks)] + \
               [("head", self.head)]

    def forward(self, latents, timestep, prompt, clip_feature=None, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        x, times, time_emb, ctx, n_img = run(self.embeddings, latents, timestep, prompt, clip_feature)
        B, S, _ = x.shape
        pf, ph, pw = c.patch_size
        grid = (latents.shape[2] // pf, latents.shape[3] // ph, latents.shape[4] // pw)
        cos, sin = ops.ref.rope3d_freqs(grid, c.hidden_size // c.num_heads, c.rope_theta, device=x.device)
        ps = get_parallel_state()
        sp = ps.enabled("ulysses")
        seq_sizes = None
        rope_full = None
        if sp:
            rope_full = (cos, sin)          # the head owner rotates its heads over the FULL sequence (fused Ulysses path)
            g = ps.get_ulysses_group()
            seq_sizes = cal_split_sizes(S, ps.size("ulysses"))
            x = split_forward_gather_backward(x, g, dim=1, grad_scale="down", split_sizes=seq_sizes)
            r = ps.rank_in("ulysses")
            st = sum(seq_sizes[:r])
            cos, sin = cos[st:st + seq_sizes[r]], sin[st:st + seq_sizes[r]]
            if len(set(seq_sizes)) == 1:
                seq_sizes = None
        if B > 1:
            cos, sin = cos.repeat(B, 1), sin.repeat(B, 1)
        for blk in self.blocks:
            x = run(blk, x, time_emb, ctx, cos, sin, seq_sizes, n_img, rope_full)
        if sp:
            x = gather_forward_split_backward(x, ps.get_ulysses_group(), dim=1, grad_scale="up",
                                              gather_sizes=cal_split_sizes(S, ps.size("ulysses")))
        y = run(self.head, x, times)
        return self.head.unpatchify(y, grid)


@model_register.register("sora")
class SoRAModel(nn.Module):
    """Generative training wrapper: (frozen AE) + (frozen text encoder) + scheduler + predictor DiT.

    With ``load_video_features / load_text_features`` the batch already carries latents and prompt
    embeddings (feature-dataset mode of the reference, mindspeed_mm/models/sora_model.py:138-222); otherwise
    ``ae`` / ``text_encoder`` callables encode under no_grad.  ``forward(batch)`` returns the weighted
    flow-matching loss; one timestep is drawn per micro-batch from ``generator``.
    """

    def __init__(self, predictor: nn.Module, scheduler, ae=None, text_encoder=None, seed: int = 0,
                 prior_loss_weight: float = 1.0):
        super().__init__()
        self.predictor, self.scheduler, self.ae, self.text_encoder = predictor, scheduler, ae, text_encoder
        self.generator = torch.Generator().manual_seed(seed)
        self.prior_loss_weight = prior_loss_weight

    def fsdp_units(self):
        return self.predictor.fsdp_units()

    def hf_ops(self):
        """Name map of the predictor's published checkpoint, when it has one (unit names carry no ``predictor.`` prefix)."""
        f = getattr(self.predictor, "hf_ops", None)
        return f() if callable(f) else None

    def forward(self, batch: dict, run=None):
        loss = self._loss(batch, run)
        if "class_video" in batch or "class_latents" in batch:
            # prior preservation (DreamBooth): the same objective on a class sample, weighted
            prior = {k[len("class_"):]: v for k, v in batch.items() if k.startswith("class_")}
            loss = loss + self.prior_loss_weight * self._loss(prior, run)
        return loss

    def _loss(self, batch: dict, run=None):
        with torch.no_grad():
            latents = batch["latents"] if "latents" in batch else self.ae.encode(batch["video"])
            prompt = batch["prompt"] if "prompt" in batch else self.text_encoder.encode(batch["prompt_ids"], batch.get("prompt_mask"))
            noise = torch.randn(latents.shape, generator=self.generator, dtype=torch.float32).to(latents.device, latents.dtype)
            x_t, noise, t = self.scheduler.q_sample(latents, noise=noise, generator=self.generator,
                                                    first_frame_latents=batch.get("first_frame_latents"))
        # fourth input: CLIP image tokens for the Wan image-to-video trunks, the prompt mask for the cross-attention DiTs
        extra = batch.get(getattr(self.predictor, "cond_input", "clip_feature"))
        pred = self.predictor(x_t, t.expand(latents.shape[0]), prompt, extra, run=run)
        loss = self.scheduler.training_losses(pred, latents, noise=noise, t=t, x_t=x_t)
        return loss.mean() if loss.dim() else loss
