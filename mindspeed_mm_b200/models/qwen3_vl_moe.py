"""Qwen3-VL-MoE style model: ViT + merger + decoder whose FFNs are top-k routed experts.

Reference behaviour (mindspeed_mm/fsdp/models/qwen3vl/modeling_qwen3_vl_moe.py:104-180): router =
``softmax(fp32) -> top-k -> renormalise -> cast``; experts stored fused as ``gate_up_proj [E, H, 2F]`` and
``down_proj [E, F, H]``; attention has per-head RMSNorm on q and k (head_dim 128) and no QKV bias.  Under
expert parallelism the experts module only holds its rank's ``E / ep`` experts and its forward is the
dispatcher in ``parallel/ep.py``; the auxiliary load-balancing loss is added when ``router_aux_loss_coef > 0``.
The vision tower reuses the windowed ViT of Qwen2.5-VL with Qwen3-VL's dimensions (patch 16, hidden 1152).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel import ep as epmod
from ..parallel.state import get_parallel_state
from .qwen2_5_vl import (Embedding, Linear, LMHead, Qwen25VLConfig, Qwen25VLModel, RMSNorm, TextConfig, VisionConfig,
                         VisionTransformer)
from .registry import model_register


@dataclass
class MoETextConfig(TextConfig):
    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    qk_norm: bool = True
    ep_dispatcher: str = "alltoall"


@dataclass
class Qwen3VLMoEConfig(Qwen25VLConfig):
    text: MoETextConfig = field(default_factory=MoETextConfig)

    @staticmethod
    def qwen3_vl_30b_a3b():
        return Qwen3VLMoEConfig(
            vision=VisionConfig(depth=27, hidden_size=1152, intermediate_size=4304, num_heads=16, patch_size=16,
                                window_size=128, fullatt_block_indexes=tuple(range(27)), out_hidden_size=2048),
            text=MoETextConfig(num_layers=48, hidden_size=2048, intermediate_size=6144, num_attention_heads=32,
                               num_key_value_heads=4, head_dim=128, vocab_size=151936, qkv_bias=False,
                               mrope_section=(24, 20, 20), num_experts=128, num_experts_per_tok=8,
                               moe_intermediate_size=768))

    @staticmethod
    def tiny():
        return Qwen3VLMoEConfig(
            vision=VisionConfig(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, fullatt_block_indexes=(1,),
                                out_hidden_size=256),
            text=MoETextConfig(num_layers=2, hidden_size=256, intermediate_size=512, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=64, vocab_size=32000, qkv_bias=False,
                               mrope_section=(8, 12, 12), num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128),
            image_token_id=31999, video_token_id=31998, vision_start_token_id=31997)


class FusedExperts(nn.Module):
    """Holds ``num_local`` experts; ``forward`` routes through the EP dispatcher when the group is > 1."""

    def __init__(self, c: MoETextConfig, num_local: Optional[int] = None):
        super().__init__()
        self.c = c
        n = num_local if num_local is not None else c.num_experts
        self.gate_up_proj = nn.Parameter(torch.empty(n, c.hidden_size, 2 * c.moe_intermediate_size))
        self.down_proj = nn.Parameter(torch.empty(n, c.moe_intermediate_size, c.hidden_size))

    def forward(self, tokens, topk_ids, probs):
        ps = get_parallel_state()
        if ps.enabled("ep"):
            kind = self.c.ep_dispatcher
            if kind in ("p2p", "mc2") and not (tokens.is_cuda and tokens.dtype == torch.bfloat16 and ops.get_tier() == "native"):
                kind = "alltoall"                      # the peer-memory dispatcher is GPU / bf16 only
            fn = {"allgather": epmod.ep_forward_allgather, "p2p": epmod.ep_forward_p2p,
                  "mc2": epmod.ep_forward_p2p}.get(kind, epmod.ep_forward_alltoall)
            return fn(tokens, topk_ids, probs, self.gate_up_proj, self.down_proj, self.c.num_experts, ps.get_ep_group())
        return ops.moe_experts(tokens, topk_ids, probs, self.gate_up_proj, self.down_proj)


class SparseMoeBlock(nn.Module):
    def __init__(self, c: MoETextConfig, num_local: Optional[int] = None):
        super().__init__()
        self.c = c
        self.gate = Linear(c.hidden_size, c.num_experts, bias=False)
        self.experts = FusedExperts(c, num_local)
        self.aux_loss = None

    def forward(self, x):
        logits = F.linear(x, self.gate.weight)                     # tiny GEMM; keep in torch
        p = torch.softmax(logits.float(), dim=-1)
        w, ids = torch.topk(p, self.c.num_experts_per_tok, dim=-1)
        if self.c.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        w = w.to(x.dtype)
        self.aux_loss = epmod.load_balancing_loss(logits, ids, self.c.num_experts) \
            if (self.c.router_aux_loss_coef > 0 and torch.is_grad_enabled()) else None
        run = getattr(self.experts, "_fsdp_run", None)
        return run(self.experts, x, ids, w) if run is not None else self.experts(x, ids, w)


class MoEDecoderLayer(nn.Module):
    def __init__(self, c: MoETextConfig, num_local: Optional[int] = None):
        super().__init__()
        self.nq, self.nkv, self.hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.qkv_proj = Linear(c.hidden_size, (self.nq + 2 * self.nkv) * self.hd, bias=c.qkv_bias)
        self.o_proj = Linear(self.nq * self.hd, c.hidden_size, bias=False)
        self.q_norm = RMSNorm(self.hd, c.rms_norm_eps) if c.qk_norm else nn.Identity()
        self.k_norm = RMSNorm(self.hd, c.rms_norm_eps) if c.qk_norm else nn.Identity()
        self.mlp = SparseMoeBlock(c, num_local)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        T = x.shape[0]
        qkv = self.qkv_proj(self.input_layernorm(x))
        q, k, v = qkv.split([self.nq * self.hd, self.nkv * self.hd, self.nkv * self.hd], dim=-1)
        q = ops.rope_rotate_half(self.q_norm(q.reshape(T, self.nq, self.hd)), cos, sin)
        k = ops.rope_rotate_half(self.k_norm(k.reshape(T, self.nkv, self.hd)), cos, sin)
        o = ops.attention_varlen(q, k, v.reshape(T, self.nkv, self.hd), cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                 causal=True)
        x = x + self.o_proj(o.reshape(T, -1))
        return x + self.mlp(self.post_attention_layernorm(x))


@model_register.register("qwen3_vl_moe")
class Qwen3VLMoEModel(Qwen25VLModel):
    def __init__(self, config: Qwen3VLMoEConfig, ep_size: Optional[int] = None):
        nn.Module.__init__(self)
        self.config = config
        t = config.text
        ep = ep_size if ep_size is not None else get_parallel_state().size("ep")
        if t.num_experts % ep:
            raise ValueError(f"num_experts {t.num_experts} must be divisible by expert_parallel_size {ep}")
        self.visual = VisionTransformer(config.vision)
        self.embed_tokens = Embedding(t.vocab_size, t.hidden_size)
        self.layers = nn.ModuleList([MoEDecoderLayer(t, t.num_experts // ep) for _ in range(t.num_layers)])
        self.lm_head = LMHead(t)

    def expert_units(self):
        """Expert parameter units (sharded over the expert-FSDP group, gradients divided by the world size)."""
        return [(f"layers.{i}.mlp.experts", l.mlp.experts) for i, l in enumerate(self.layers)]

    def aux_loss(self):
        ls = [l.mlp.aux_loss for l in self.layers if l.mlp.aux_loss is not None]
        return self.config.text.router_aux_loss_coef * torch.stack(ls).mean() if ls else None
