"""Frozen prompt encoders for the generative models: T5 / umT5 encoder and CLIP text transformer.

The reference wraps HuggingFace classes behind one ``TextEncoder`` facade
(mindspeed_mm/models/text_encoder/text_encoder.py:31) and calls ``encode(input_ids, mask)`` under no_grad from
``SoRAModel.forward`` (mindspeed_mm/models/sora_model.py:154-171).  Here the encoders are written out so that their
linears and attention run through :mod:`mindspeed_mm_b200.ops` (tcgen05 GEMM / FMHA on a GPU), and they load HF
checkpoints by name map (``hf_name_map``).

* ``T5Encoder``: pre-norm RMSNorm blocks, un-scaled attention with a learned relative-position bias
  (shared across layers for T5, one table per layer for umT5), gated-GELU feed-forward.
* ``CLIPTextEncoder``: causal pre-LN transformer with learned positions; returns the hidden states and the
  pooled state at the end-of-text token.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


# ------------------------------------------------------------------------------------------ T5 / umT5
@dataclass
class T5Config:
    vocab_size: int = 256384
    d_model: int = 4096
    d_kv: int = 64
    d_ff: int = 10240
    num_layers: int = 24
    num_heads: int = 64
    num_buckets: int = 32
    max_distance: int = 128
    per_layer_bias: bool = True       # umT5: every layer owns a relative-position table
    gated: bool = True                # gated-GELU (v1.1 / umT5) or plain ReLU (original T5)
    eps: float = 1e-6

    @classmethod
    def umt5_xxl(cls):
        return cls()

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4), **kw})


def relative_position_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional T5 bucketing: half of the buckets for each sign, exact below ``max_exact``, log-spaced above."""
    nb = num_buckets // 2
    out = (rel > 0).long() * nb
    n = rel.abs()
    max_exact = nb // 2
    large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact)
                         * (nb - max_exact)).long()
    large = large.clamp(max=nb - 1)
    return out + torch.where(n < max_exact, n, large)


class T5Attention(nn.Module):
    def __init__(self, c: T5Config, has_bias_table: bool):
        super().__init__()
        inner = c.num_heads * c.d_kv
        self.c = c
        self.q = nn.Linear(c.d_model, inner, bias=False)
        self.k = nn.Linear(c.d_model, inner, bias=False)
        self.v = nn.Linear(c.d_model, inner, bias=False)
        self.o = nn.Linear(inner, c.d_model, bias=False)
        self.relative_attention_bias = nn.Embedding(c.num_buckets, c.num_heads) if has_bias_table else None

    def position_bias(self, L: int, device) -> torch.Tensor:
        pos = torch.arange(L, device=device)
        bucket = relative_position_bucket(pos[None, :] - pos[:, None], self.c.num_buckets, self.c.max_distance)
        return self.relative_attention_bias(bucket).permute(2, 0, 1)          # [N, L, L]

    def forward(self, x, bias):
        B, L, _ = x.shape
        N, D = self.c.num_heads, self.c.d_kv
        q = ops.linear(x, self.q.weight).view(B, L, N, D).transpose(1, 2)
        k = ops.linear(x, self.k.weight).view(B, L, N, D).transpose(1, 2)
        v = ops.linear(x, self.v.weight).view(B, L, N, D).transpose(1, 2)
        # additive bias -> score path in torch (T5 does not scale by 1/sqrt(d)); prompts are <= 512 tokens
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) + bias
        p = torch.softmax(s, -1).to(v.dtype)
        o = torch.matmul(p, v).transpose(1, 2).reshape(B, L, N * D)
        return ops.linear(o, self.o.weight)


class T5Block(nn.Module):
    def __init__(self, c: T5Config, has_bias_table: bool):
        super().__init__()
        self.c = c
        self.norm1 = nn.Parameter(torch.ones(c.d_model))
        self.attn = T5Attention(c, has_bias_table)
        self.norm2 = nn.Parameter(torch.ones(c.d_model))
        if c.gated:
            self.wi_0 = nn.Linear(c.d_model, c.d_ff, bias=False)
            self.wi_1 = nn.Linear(c.d_model, c.d_ff, bias=False)
        else:
            self.wi = nn.Linear(c.d_model, c.d_ff, bias=False)
        self.wo = nn.Linear(c.d_ff, c.d_model, bias=False)

    def forward(self, x, bias):
        x = x + self.attn(ops.rms_norm(x, self.norm1, self.c.eps), bias)
        h = ops.rms_norm(x, self.norm2, self.c.eps)
        if self.c.gated:
            h = ops.gelu_tanh(ops.linear(h, self.wi_0.weight)) * ops.linear(h, self.wi_1.weight)
        else:
            h = F.relu(ops.linear(h, self.wi.weight))
        return x + ops.linear(h, self.wo.weight)


class T5Encoder(nn.Module):
    def __init__(self, c: T5Config):
        super().__init__()
        self.c = c
        self.embed = nn.Embedding(c.vocab_size, c.d_model)
        self.blocks = nn.ModuleList(T5Block(c, c.per_layer_bias or i == 0) for i in range(c.num_layers))
        self.final_norm = nn.Parameter(torch.ones(c.d_model))

    def forward(self, input_ids, attention_mask=None):
        x = self.embed(input_ids)
        B, L = input_ids.shape
        pad = None
        if attention_mask is not None:
            pad = (1.0 - attention_mask[:, None, None, :].float()) * torch.finfo(torch.float32).min
        bias = None
        for blk in self.blocks:
            if blk.attn.relative_attention_bias is not None:
                bias = blk.attn.position_bias(L, x.device).float()[None]
                if pad is not None:
                    bias = bias + pad
            x = blk(x, bias)
        return ops.rms_norm(x, self.final_norm, self.c.eps)

    @torch.no_grad()
    def encode(self, input_ids, attention_mask=None):
        """Prompt embeddings with padded positions zeroed (what the Wan pipeline feeds the DiT)."""
        h = self(input_ids, attention_mask)
        return h if attention_mask is None else h * attention_mask[..., None].to(h.dtype)

    def hf_name_map(self) -> Dict[str, str]:
        """this module's parameter name -> ``UMT5EncoderModel`` / ``T5EncoderModel`` state-dict name."""
        m = {"embed.weight": "shared.weight", "final_norm": "encoder.final_layer_norm.weight"}
        for i, blk in enumerate(self.blocks):
            a, f = f"encoder.block.{i}.layer.0", f"encoder.block.{i}.layer.1"
            for n in "qkvo":
                m[f"blocks.{i}.attn.{n}.weight"] = f"{a}.SelfAttention.{n}.weight"
            if blk.attn.relative_attention_bias is not None:
                m[f"blocks.{i}.attn.relative_attention_bias.weight"] = f"{a}.SelfAttention.relative_attention_bias.weight"
            m[f"blocks.{i}.norm1"] = f"{a}.layer_norm.weight"
            m[f"blocks.{i}.norm2"] = f"{f}.layer_norm.weight"
            for n in (("wi_0", "wi_1") if self.c.gated else ("wi",)):
                m[f"blocks.{i}.{n}.weight"] = f"{f}.DenseReluDense.{n}.weight"
            m[f"blocks.{i}.wo.weight"] = f"{f}.DenseReluDense.wo.weight"
        return m

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        own = dict(self.named_parameters())
        for mine, theirs in self.hf_name_map().items():
            own[mine].data.copy_(sd[theirs])


# ------------------------------------------------------------------------------------------ CLIP text
@dataclass
class CLIPTextConfig:
    vocab_size: int = 49408
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_layers: int = 12
    num_heads: int = 12
    max_positions: int = 77
    eos_token_id: int = 49407
    act: str = "quick_gelu"
    eps: float = 1e-5

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(vocab_size=100, hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4,
                             max_positions=16, eos_token_id=99), **kw})


def _act(name: str, x):
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name == "gelu":
        return ops.gelu(x)
    return ops.gelu_tanh(x)


class CLIPLayer(nn.Module):
    def __init__(self, hidden, inter, heads, act, eps):
        super().__init__()
        self.heads, self.act, self.eps = heads, act, eps
        self.ln1 = ops.LayerNorm(hidden, eps=eps)
        self.qkv = nn.Linear(hidden, 3 * hidden)
        self.out = nn.Linear(hidden, hidden)
        self.ln2 = ops.LayerNorm(hidden, eps=eps)
        self.fc1 = nn.Linear(hidden, inter)
        self.fc2 = nn.Linear(inter, hidden)

    def forward(self, x, causal: bool):
        B, L, H = x.shape
        qkv = ops.linear(self.ln1(x), self.qkv.weight, self.qkv.bias).view(B, L, 3, self.heads, H // self.heads)
        o = ops.attention_dense(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=causal)
        x = x + ops.linear(o.reshape(B, L, H), self.out.weight, self.out.bias)
        h = _act(self.act, ops.linear(self.ln2(x), self.fc1.weight, self.fc1.bias))
        return x + ops.linear(h, self.fc2.weight, self.fc2.bias)


class CLIPTextEncoder(nn.Module):
    def __init__(self, c: CLIPTextConfig):
        super().__init__()
        self.c = c
        self.token_embedding = nn.Embedding(c.vocab_size, c.hidden_size)
        self.position_embedding = nn.Embedding(c.max_positions, c.hidden_size)
        self.layers = nn.ModuleList(CLIPLayer(c.hidden_size, c.intermediate_size, c.num_heads, c.act, c.eps)
                                    for _ in range(c.num_layers))
        self.final_ln = ops.LayerNorm(c.hidden_size, eps=c.eps)

    def forward(self, input_ids):
        B, L = input_ids.shape
        x = self.token_embedding(input_ids) + self.position_embedding.weight[:L]
        for layer in self.layers:
            x = layer(x, causal=True)
        x = self.final_ln(x)
        eos = (input_ids == self.c.eos_token_id).int().argmax(-1)
        return x, x[torch.arange(B, device=x.device), eos]

    @torch.no_grad()
    def encode(self, input_ids, attention_mask=None):
        return self(input_ids)[1]

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], prefix: str = "text_model.") -> None:
        """Loads ``CLIPTextModel`` weights; q/k/v projections are fused into one ``qkv`` here."""
        g = lambda k: sd[prefix + k]
        self.token_embedding.weight.data.copy_(g("embeddings.token_embedding.weight"))
        self.position_embedding.weight.data.copy_(g("embeddings.position_embedding.weight"))
        for i, l in enumerate(self.layers):
            p = f"encoder.layers.{i}."
            for kind in ("weight", "bias"):
                getattr(l.qkv, kind).data.copy_(torch.cat([g(p + f"self_attn.{n}_proj.{kind}") for n in "qkv"], 0))
                getattr(l.out, kind).data.copy_(g(p + f"self_attn.out_proj.{kind}"))
                getattr(l.ln1, kind).data.copy_(g(p + f"layer_norm1.{kind}"))
                getattr(l.ln2, kind).data.copy_(g(p + f"layer_norm2.{kind}"))
                getattr(l.fc1, kind).data.copy_(g(p + f"mlp.fc1.{kind}"))
                getattr(l.fc2, kind).data.copy_(g(p + f"mlp.fc2.{kind}"))
        for kind in ("weight", "bias"):
            getattr(self.final_ln, kind).data.copy_(g(f"final_layer_norm.{kind}"))


class TextEncoder(nn.Module):
    """Facade over one or several encoders (the reference accepts a list for dual-encoder models such as
    HunyuanVideo / FLUX: text_encoder.py:31).  ``encode`` returns one tensor or a list in the same order."""

    def __init__(self, encoders):
        super().__init__()
        self.single = isinstance(encoders, nn.Module)
        self.encoders = nn.ModuleList([encoders] if self.single else list(encoders))
        for p in self.parameters():
            p.requires_grad_(False)

    @torch.no_grad()
    def encode(self, input_ids, attention_mask=None):
        if self.single:
            return self.encoders[0].encode(input_ids, attention_mask)
        masks = attention_mask if isinstance(attention_mask, (list, tuple)) else [attention_mask] * len(self.encoders)
        return [e.encode(i, m) for e, i, m in zip(self.encoders, input_ids, masks)]
