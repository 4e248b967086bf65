"""Qwen3.5-style hybrid decoder: gated-delta-net (GDN) linear-attention layers with a full-attention layer every
``full_attention_interval`` layers, on packed sequences.

GDN layer (mindspeed_mm/fsdp/models/qwen3_5_moe/modeling_qwen3_5_moe.py:337-360,530-915): fused input projection
to q | k | v | z | b | a; depthwise causal conv (kernel 4) + SiLU on q, k, v; q and k L2-normalised per head;
``beta = sigmoid(b)``, ``g = -exp(A_log) * softplus(a + dt_bias)``; chunked gated delta rule (chunk 64);
``rmsnorm(o) * weight * silu(z)``; output projection.  Sequences never mix: the conv and the recurrence restart at
every ``cu_seqlens`` boundary.  The vision tower / merger / embedding / head are those of the Qwen2.5-VL model.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .qwen2_5_vl import (DecoderLayer, Embedding, Linear, LMHead, Qwen25VLConfig, Qwen25VLModel, RMSNorm, TextConfig,
                         VisionConfig, VisionTransformer)
from .registry import model_register


@dataclass
class GDNTextConfig(TextConfig):
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    full_attention_interval: int = 4
    gdn_chunk: int = 64


@dataclass
class Qwen35Config(Qwen25VLConfig):
    text: GDNTextConfig = field(default_factory=GDNTextConfig)

    @staticmethod
    def tiny():
        return Qwen35Config(
            vision=VisionConfig(depth=1, hidden_size=128, intermediate_size=256, num_heads=4, fullatt_block_indexes=(0,),
                                out_hidden_size=256),
            text=GDNTextConfig(num_layers=4, hidden_size=256, intermediate_size=512, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=64, vocab_size=32000, qkv_bias=False, mrope_section=(8, 12, 12),
                               linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
                               linear_value_head_dim=32, full_attention_interval=4, gdn_chunk=16),
            image_token_id=31999, video_token_id=31998, vision_start_token_id=31997)


class GatedDeltaNet(nn.Module):
    def __init__(self, c: GDNTextConfig):
        super().__init__()
        self.c = c
        self.hk, self.hv, self.dk, self.dv = c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        self.conv_dim = 2 * self.key_dim + self.value_dim
        # q | k | v | z | b | a
        self.in_proj = Linear(c.hidden_size, self.conv_dim + self.value_dim + 2 * self.hv, bias=False)
        self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, c.linear_conv_kernel_dim))
        self.A_log = nn.Parameter(torch.zeros(self.hv))
        self.dt_bias = nn.Parameter(torch.zeros(self.hv))
        self.norm_weight = nn.Parameter(torch.ones(self.dv))
        self.out_proj = Linear(self.value_dim, c.hidden_size, bias=False)

    def post_init(self):
        with torch.no_grad():
            self.A_log.copy_(torch.log(torch.linspace(1.0, 8.0, self.hv)))
            self.dt_bias.zero_()
            self.norm_weight.fill_(1.0)
            self.conv_weight.normal_(0.0, 0.2)

    def forward(self, x, cu_seqlens):
        T = x.shape[0]
        proj = self.in_proj(x)
        qkv, z, b, a = proj.split([self.conv_dim, self.value_dim, self.hv, self.hv], dim=-1)
        qkv = ops.causal_conv1d(qkv, self.conv_weight.to(qkv.dtype), None, "silu", cu_seqlens)
        q, k, v = qkv.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        rep = self.hv // self.hk
        q = ops.l2_norm(q.reshape(T, self.hk, self.dk)).repeat_interleave(rep, dim=1)
        k = ops.l2_norm(k.reshape(T, self.hk, self.dk)).repeat_interleave(rep, dim=1)
        v = v.reshape(T, self.hv, self.dv)
        beta = torch.sigmoid(b.float())
        g = -torch.exp(self.A_log.float()) * F.softplus(a.float() + self.dt_bias.float())
        o = ops.gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, chunk=self.c.gdn_chunk)
        o = ops.gated_rms_norm(o.to(x.dtype), z.reshape(T, self.hv, self.dv), self.norm_weight, self.c.rms_norm_eps)
        return self.out_proj(o.reshape(T, self.value_dim))


class GDNDecoderLayer(nn.Module):
    def __init__(self, c: GDNTextConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.linear_attn = GatedDeltaNet(c)
        self.gate_up_proj = Linear(c.hidden_size, 2 * c.intermediate_size, bias=False)
        self.down_proj = Linear(c.intermediate_size, c.hidden_size, bias=False)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        x = x + self.linear_attn(self.input_layernorm(x), cu_seqlens)
        return x + self.down_proj(ops.linear_swiglu(self.post_attention_layernorm(x), self.gate_up_proj.weight))


@model_register.register("qwen3_5")
class Qwen35Model(Qwen25VLModel):
    def __init__(self, config: Qwen35Config):
        nn.Module.__init__(self)
        self.config = config
        t = config.text
        self.visual = VisionTransformer(config.vision)
        self.embed_tokens = Embedding(t.vocab_size, t.hidden_size)
        self.layers = nn.ModuleList([
            DecoderLayer(t) if (i + 1) % t.full_attention_interval == 0 else GDNDecoderLayer(t) for i in range(t.num_layers)])
        self.lm_head = LMHead(t)
