"""Stand-alone image and audio encoders used as conditioning towers.

* ``CLIPVisionEncoder`` -- pre-LN ViT with a class token (CLIP / open-CLIP ViT-H as used for Wan image-to-video
  conditioning, mindspeed_mm/models/vision/vision_encoders/clip_vit_model.py; Wan I2V takes the penultimate
  layer's hidden states, mindspeed_mm/utils/extra_processor/wan_i2v_processor.py).
* ``WhisperEncoder`` -- two strided 1-D convolutions over log-mel frames, fixed sinusoidal positions, pre-LN
  transformer (mindspeed_mm/models/whisper/whisper_model.py; the Qwen2.5-Omni audio tower,
  mindspeed_mm/models/audio/, is the same encoder run over fixed-length windows with block-diagonal attention and a
  2x average pool + projection on top -- ``WindowedAudioEncoder``).

Linears and attention go through :mod:`mindspeed_mm_b200.ops`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .text_encoder import CLIPLayer


# ------------------------------------------------------------------------------------------ CLIP vision
@dataclass
class CLIPVisionConfig:
    image_size: int = 224
    patch_size: int = 14
    hidden_size: int = 1280
    intermediate_size: int = 5120
    num_layers: int = 32
    num_heads: int = 16
    act: str = "gelu"
    eps: float = 1e-5

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(image_size=28, patch_size=14, hidden_size=64, intermediate_size=128, num_layers=3,
                             num_heads=4, act="quick_gelu"), **kw})


class CLIPVisionEncoder(nn.Module):
    def __init__(self, c: CLIPVisionConfig):
        super().__init__()
        self.c = c
        n = (c.image_size // c.patch_size) ** 2
        self.class_embedding = nn.Parameter(torch.zeros(c.hidden_size))
        self.patch_embedding = nn.Conv2d(3, c.hidden_size, c.patch_size, stride=c.patch_size, bias=False)
        self.position_embedding = nn.Embedding(n + 1, c.hidden_size)
        self.pre_ln = ops.LayerNorm(c.hidden_size, eps=c.eps)
        self.layers = nn.ModuleList(CLIPLayer(c.hidden_size, c.intermediate_size, c.num_heads, c.act, c.eps)
                                    for _ in range(c.num_layers))
        self.post_ln = ops.LayerNorm(c.hidden_size, eps=c.eps)

    def forward(self, pixels, output_layer: int = -1):
        """pixels [B,3,H,W] -> (hidden states of layer ``output_layer`` [B,1+N,H], pooled class token)."""
        B = pixels.shape[0]
        x = self.patch_embedding(pixels).flatten(2).transpose(1, 2)
        x = torch.cat([self.class_embedding.expand(B, 1, -1).to(x.dtype), x], dim=1) + self.position_embedding.weight
        x = self.pre_ln(x)
        n = len(self.layers)
        stop = n if output_layer == -1 else (n + 1 + output_layer if output_layer < 0 else output_layer)
        for layer in self.layers[:stop]:
            x = layer(x, causal=False)
        return x, self.post_ln(x[:, 0])

    @torch.no_grad()
    def encode(self, pixels):
        """Penultimate-layer tokens: the image conditioning of Wan I2V."""
        return self(pixels, output_layer=-2)[0]

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], prefix: str = "vision_model.") -> None:
        g = lambda k: sd[prefix + k]
        self.class_embedding.data.copy_(g("embeddings.class_embedding"))
        self.patch_embedding.weight.data.copy_(g("embeddings.patch_embedding.weight"))
        self.position_embedding.weight.data.copy_(g("embeddings.position_embedding.weight"))
        for kind in ("weight", "bias"):
            getattr(self.pre_ln, kind).data.copy_(g(f"pre_layrnorm.{kind}"))
            getattr(self.post_ln, kind).data.copy_(g(f"post_layernorm.{kind}"))
        for i, l in enumerate(self.layers):
            p = f"encoder.layers.{i}."
            for kind in ("weight", "bias"):
                getattr(l.qkv, kind).data.copy_(torch.cat([g(p + f"self_attn.{n}_proj.{kind}") for n in "qkv"], 0))
                getattr(l.out, kind).data.copy_(g(p + f"self_attn.out_proj.{kind}"))
                getattr(l.ln1, kind).data.copy_(g(p + f"layer_norm1.{kind}"))
                getattr(l.ln2, kind).data.copy_(g(p + f"layer_norm2.{kind}"))
                getattr(l.fc1, kind).data.copy_(g(p + f"mlp.fc1.{kind}"))
                getattr(l.fc2, kind).data.copy_(g(p + f"mlp.fc2.{kind}"))


# ------------------------------------------------------------------------------------------ audio
@dataclass
class WhisperConfig:
    num_mel_bins: int = 128
    d_model: int = 1280
    ffn_dim: int = 5120
    num_layers: int = 32
    num_heads: int = 20
    max_source_positions: int = 1500
    eps: float = 1e-5

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(num_mel_bins=16, d_model=64, ffn_dim=128, num_layers=2, num_heads=4,
                             max_source_positions=50), **kw})


def sinusoid_positions(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2))
    t = torch.arange(length)[:, None] * inv[None]
    return torch.cat([t.sin(), t.cos()], dim=1)


class WhisperLayer(nn.Module):
    def __init__(self, c: WhisperConfig):
        super().__init__()
        self.heads = c.num_heads
        d = c.d_model
        self.ln1 = ops.LayerNorm(d, eps=c.eps)
        self.q = nn.Linear(d, d)
        self.k = nn.Linear(d, d, bias=False)
        self.v = nn.Linear(d, d)
        self.out = nn.Linear(d, d)
        self.ln2 = ops.LayerNorm(d, eps=c.eps)
        self.fc1 = nn.Linear(d, c.ffn_dim)
        self.fc2 = nn.Linear(c.ffn_dim, d)

    def forward(self, x, cu_seqlens, max_len):
        """x: packed [T, d]; attention is confined to the ``cu_seqlens`` segments."""
        T, d = x.shape
        h = self.ln1(x)
        q = ops.linear(h, self.q.weight, self.q.bias).view(T, self.heads, -1)
        k = ops.linear(h, self.k.weight).view(T, self.heads, -1)
        v = ops.linear(h, self.v.weight, self.v.bias).view(T, self.heads, -1)
        o = ops.attention_varlen(q, k, v, cu_seqlens, cu_seqlens, max_len, max_len, causal=False)
        x = x + ops.linear(o.reshape(T, d), self.out.weight, self.out.bias)
        return x + ops.linear(ops.gelu(ops.linear(self.ln2(x), self.fc1.weight, self.fc1.bias)), self.fc2.weight, self.fc2.bias)


class WhisperEncoder(nn.Module):
    def __init__(self, c: WhisperConfig):
        super().__init__()
        self.c = c
        self.conv1 = nn.Conv1d(c.num_mel_bins, c.d_model, 3, padding=1)
        self.conv2 = nn.Conv1d(c.d_model, c.d_model, 3, stride=2, padding=1)
        # the sinusoid table is computed on demand: a buffer would stay on the meta device when the model is built there
        self._positions: dict = {}
        self.layers = nn.ModuleList(WhisperLayer(c) for _ in range(c.num_layers))
        self.ln_post = ops.LayerNorm(c.d_model, eps=c.eps)

    def embed(self, mel):
        """mel [B, n_mels, frames] -> [B, frames/2, d] with positions added."""
        x = ops.gelu(self.conv1(mel))
        x = ops.gelu(self.conv2(x)).transpose(1, 2)
        key = (x.device, x.dtype)
        if key not in self._positions:
            base = getattr(self, "_loaded_positions", None)
            base = base if base is not None else sinusoid_positions(self.c.max_source_positions, self.c.d_model)
            self._positions[key] = base.to(x.device, x.dtype)
        return x + self._positions[key][: x.shape[1]]

    def forward(self, mel):
        x = self.embed(mel)
        B, L, d = x.shape
        cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=x.device)
        x = x.reshape(B * L, d)
        for layer in self.layers:
            x = layer(x, cu, L)
        return self.ln_post(x).view(B, L, d)

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], prefix: str = "encoder.") -> None:
        g = lambda k: sd[prefix + k]
        for n in ("conv1", "conv2"):
            getattr(self, n).weight.data.copy_(g(f"{n}.weight"))
            getattr(self, n).bias.data.copy_(g(f"{n}.bias"))
        table = g("embed_positions.weight")               # the published table (the same sinusoids) replaces the computed one
        self._positions = {(table.device, table.dtype): table.clone()}
        self._loaded_positions = table.clone()
        for kind in ("weight", "bias"):
            getattr(self.ln_post, kind).data.copy_(g(f"layer_norm.{kind}"))
        for i, l in enumerate(self.layers):
            p = f"layers.{i}."
            for mine, theirs in (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"),
                                 ("out", "self_attn.out_proj"), ("ln1", "self_attn_layer_norm"),
                                 ("ln2", "final_layer_norm"), ("fc1", "fc1"), ("fc2", "fc2")):
                mod = getattr(l, mine)
                mod.weight.data.copy_(g(p + theirs + ".weight"))
                if mod.bias is not None:
                    mod.bias.data.copy_(g(p + theirs + ".bias"))


class WindowedAudioEncoder(nn.Module):
    """Omni-style audio tower: the mel stream is cut into windows of ``2 * n_window`` frames, each window is
    embedded on its own (conv + positions restart per window), all windows of all clips are packed into one
    token stream with block-diagonal attention, then 2x average-pooled and projected to the LLM width."""

    def __init__(self, c: WhisperConfig, n_window: int = 100, output_dim: int = 3584):
        super().__init__()
        self.enc = WhisperEncoder(c)
        self.n_window = n_window
        self.proj = nn.Linear(c.d_model, output_dim)

    def forward(self, mels: List[torch.Tensor]):
        """mels: list of [n_mels, frames_i].  Returns the list of [ceil(frames_i / 4), output_dim] embeddings."""
        win = 2 * self.n_window
        chunks, owners = [], []
        for i, m in enumerate(mels):
            for s in range(0, m.shape[1], win):
                chunks.append(m[:, s:s + win])
                owners.append(i)
        embs = [self.enc.embed(ch[None])[0] for ch in chunks]               # [len_j, d]
        lens = [e.shape[0] for e in embs]
        x = torch.cat(embs, 0)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=x.device)
        for layer in self.enc.layers:
            x = layer(x, cu, max(lens))
        outs: List[List[torch.Tensor]] = [[] for _ in mels]
        for i, seg in zip(owners, x.split(lens, 0)):
            outs[i].append(seg)
        res = []
        for segs in outs:
            h = torch.cat(segs, 0)
            if h.shape[0] % 2:
                h = h[:-1] if h.shape[0] > 1 else torch.cat([h, h], 0)
            h = h.view(-1, 2, h.shape[-1]).mean(1)
            res.append(ops.linear(self.enc.ln_post(h), self.proj.weight, self.proj.bias))
        return res
