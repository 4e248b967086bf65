"""Qwen3.5 (dense and MoE): hybrid decoder of gated-delta-net (GDN) linear-attention layers with a gated full-attention
layer every ``full_attention_interval`` layers, behind the Qwen3-VL vision tower (no DeepStack), on packed sequences.

Reference: mindspeed_mm/fsdp/models/qwen3_5_moe/modeling_qwen3_5_moe.py:337-360,530-915 and the upstream Hugging Face
modeling it derives from.

* GDN layer: input projection to q | k | v | z | b | a; depthwise causal conv (kernel 4) + SiLU on q, k, v; q and k
  L2-normalised per head; ``beta = sigmoid(b)``, ``g = -exp(A_log) * softplus(a + dt_bias)``; chunked gated delta rule
  (chunk 64, queries scaled by ``1 / sqrt(d_k)``); ``rmsnorm(o) * weight * silu(z)``; output projection.  Sequences never
  mix: the conv and the recurrence restart at every ``cu_seqlens`` boundary.
* full-attention layer: the query projection is twice as wide (per head: query | gate), per-head q/k RMSNorm, rotary
  embedding on the first ``partial_rotary_factor`` of the head dim (interleaved mRoPE bands), and the attention output
  is multiplied by ``sigmoid(gate)`` before the output projection.
* every RMSNorm of the text stack is stored here as the usual multiplicative weight; Hugging Face stores ``weight - 1``
  (zero-centred), which the weight map adds back and removes (``checkpoint/hf.py: qwen35_ops``).
* MoE variant: ``softmax -> top-k -> renormalise`` routed experts plus a shared expert scaled by
  ``sigmoid(shared_expert_gate(x))``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel.state import get_parallel_state
from .moe import MoETextConfig, SparseMoeBlock
from .qwen2_5_vl import Embedding, Linear, LMHead, RMSNorm, TextConfig, _normal_like
from .qwen3_vl import (Qwen3VisionConfig, Qwen3VisionTransformer, interleaved_mrope_cos_sin, qwen3_rope_index,
                       qwen3_vision_plan)
from .registry import model_register


@dataclass
class GDNTextConfig(TextConfig):
    """The linear-attention fields (also read by the composable decoder's GDN mixer)."""
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    full_attention_interval: int = 4
    gdn_chunk: int = 64


@dataclass
class Qwen35TextConfig(MoETextConfig, GDNTextConfig):
    qkv_bias: bool = False
    head_dim: Optional[int] = 256
    rope_theta: float = 1e7
    mrope_section: Sequence[int] = (11, 11, 10)
    partial_rotary_factor: float = 0.25
    attn_output_gate: bool = True
    num_experts: int = 0                       # 0: dense SwiGLU FFN
    shared_expert_intermediate_size: int = 0
    mtp_num_layers: int = 0                    # multi-token prediction: extra full-attention layer(s) predicting token t + 2
    mtp_loss_scaling_factor: float = 0.1

    def layer_is_linear(self, i: int) -> bool:
        return (i + 1) % self.full_attention_interval != 0


@dataclass
class Qwen35Config:
    vision: Qwen3VisionConfig = field(default_factory=lambda: Qwen3VisionConfig(deepstack_visual_indexes=(), out_hidden_size=4096))
    text: Qwen35TextConfig = field(default_factory=Qwen35TextConfig)
    image_token_id: int = 248056
    video_token_id: int = 248057
    vision_start_token_id: int = 248053
    vision_end_token_id: int = 248054
    init_std: float = 0.02

    def vision_plan(self, grid_thw: torch.Tensor) -> dict:
        return qwen3_vision_plan(self.vision, grid_thw)

    def rope_index(self, input_ids: torch.Tensor, image_grid_thw=None, video_grid_thw=None):
        return qwen3_rope_index(input_ids, image_grid_thw, video_grid_thw, self.image_token_id, self.video_token_id,
                                self.vision.spatial_merge_size)

    @staticmethod
    def qwen3_5_9b():
        return Qwen35Config(text=Qwen35TextConfig(num_layers=32, hidden_size=4096, intermediate_size=12288, num_attention_heads=16,
                                               num_key_value_heads=4, vocab_size=248320))

    @staticmethod
    def qwen3_5_35b_a3b():
        return Qwen35Config(
            vision=Qwen3VisionConfig(deepstack_visual_indexes=(), out_hidden_size=2048),
            text=Qwen35TextConfig(num_layers=40, hidden_size=2048, intermediate_size=0, num_attention_heads=16,
                               num_key_value_heads=2, vocab_size=248320, num_experts=256, num_experts_per_tok=8,
                               moe_intermediate_size=512, shared_expert_intermediate_size=512))

    @staticmethod
    def tiny(moe: bool = False):
        return Qwen35Config(
            vision=Qwen3VisionConfig(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, out_hidden_size=256,
                                     num_position_embeddings=64, deepstack_visual_indexes=()),
            text=Qwen35TextConfig(num_layers=4, hidden_size=256, intermediate_size=512, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=64, vocab_size=32000, mrope_section=(3, 3, 2),
                               linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
                               linear_value_head_dim=32, full_attention_interval=4, gdn_chunk=16,
                               num_experts=8 if moe else 0, num_experts_per_tok=2, moe_intermediate_size=128,
                               shared_expert_intermediate_size=128 if moe else 0),
            image_token_id=31999, video_token_id=31998, vision_start_token_id=31997, vision_end_token_id=31996)

    @staticmethod
    def from_hf(hf: dict) -> "Qwen35Config":
        """From a Hugging Face ``config.json`` (``qwen3_5`` / ``qwen3_5_moe``)."""
        v, t = hf.get("vision_config", {}), hf.get("text_config", hf)
        rp = t.get("rope_parameters") or {}
        types = t.get("layer_types")
        interval = t.get("full_attention_interval") or (types.index("full_attention") + 1 if types else 4)
        vis = Qwen3VisionConfig(
            depth=v.get("depth", 27), hidden_size=v.get("hidden_size", 1152), intermediate_size=v.get("intermediate_size", 4304),
            num_heads=v.get("num_heads", 16), in_channels=v.get("in_channels", 3), patch_size=v.get("patch_size", 16),
            temporal_patch_size=v.get("temporal_patch_size", 2), spatial_merge_size=v.get("spatial_merge_size", 2),
            out_hidden_size=v.get("out_hidden_size", t["hidden_size"]),
            num_position_embeddings=v.get("num_position_embeddings", 2304), deepstack_visual_indexes=())
        txt = Qwen35TextConfig(
            num_layers=t["num_hidden_layers"], hidden_size=t["hidden_size"], intermediate_size=t.get("intermediate_size", 0),
            num_attention_heads=t["num_attention_heads"], num_key_value_heads=t["num_key_value_heads"],
            head_dim=t.get("head_dim") or t["hidden_size"] // t["num_attention_heads"], vocab_size=t["vocab_size"],
            rms_norm_eps=t.get("rms_norm_eps", 1e-6), rope_theta=rp.get("rope_theta", 1e7),
            mrope_section=tuple(rp.get("mrope_section", (11, 11, 10))),
            partial_rotary_factor=rp.get("partial_rotary_factor", t.get("partial_rotary_factor", 0.25)),
            qkv_bias=t.get("attention_bias", False), linear_num_key_heads=t["linear_num_key_heads"],
            linear_num_value_heads=t["linear_num_value_heads"], linear_key_head_dim=t["linear_key_head_dim"],
            linear_value_head_dim=t["linear_value_head_dim"], linear_conv_kernel_dim=t.get("linear_conv_kernel_dim", 4),
            full_attention_interval=interval, num_experts=t.get("num_experts", t.get("num_local_experts", 0)),
            num_experts_per_tok=t.get("num_experts_per_tok", 8), moe_intermediate_size=t.get("moe_intermediate_size", 512),
            shared_expert_intermediate_size=t.get("shared_expert_intermediate_size", 0),
            router_aux_loss_coef=t.get("router_aux_loss_coef", 0.0),
            tie_word_embeddings=hf.get("tie_word_embeddings", t.get("tie_word_embeddings", False)))
        return Qwen35Config(vision=vis, text=txt, image_token_id=hf.get("image_token_id", 248056),
                            video_token_id=hf.get("video_token_id", 248057),
                            vision_start_token_id=hf.get("vision_start_token_id", 248053),
                            vision_end_token_id=hf.get("vision_end_token_id", 248054))


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
        o = ops.gated_rms_norm(o, z.reshape(T, self.hv, self.dv), self.norm_weight, self.c.rms_norm_eps)      # fp32 in, z's dtype out
        return self.out_proj(o.reshape(T, self.value_dim))


class GatedAttention(nn.Module):
    """Full attention of the hybrid stack: query | gate projection, q/k norm, partial rotary, sigmoid output gate."""

    def __init__(self, c: Qwen35TextConfig):
        super().__init__()
        self.nq, self.nkv, self.hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        self.gated = c.attn_output_gate
        self.rot = int(c.head_dim * c.partial_rotary_factor)
        # rows per head: query then gate (the checkpoint layout of q_proj), then all keys, then all values
        self.qkv_proj = Linear(c.hidden_size, (self.nq * (2 if self.gated else 1) + 2 * self.nkv) * self.hd, bias=c.qkv_bias)
        self.o_proj = Linear(self.nq * self.hd, c.hidden_size, bias=c.qkv_bias)
        self.q_norm = RMSNorm(self.hd, c.rms_norm_eps)
        self.k_norm = RMSNorm(self.hd, c.rms_norm_eps)

    def _rope(self, x, cos, sin):
        if self.rot == self.hd:
            return ops.rope_rotate_half(x, cos, sin)
        return torch.cat([ops.rope_rotate_half(x[..., :self.rot].contiguous(), cos, sin), x[..., self.rot:]], dim=-1)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen, cache: Optional[dict] = None):
        T = x.shape[0]
        qw = self.nq * self.hd * (2 if self.gated else 1)
        q, k, v = self.qkv_proj(x).split([qw, self.nkv * self.hd, self.nkv * self.hd], dim=-1)
        gate = None
        if self.gated:
            q, gate = q.reshape(T, self.nq, 2 * self.hd).chunk(2, dim=-1)
            gate = gate.reshape(T, self.nq * self.hd)
        q = self._rope(self.q_norm(q.reshape(T, self.nq, self.hd)), cos, sin)
        k = self._rope(self.k_norm(k.reshape(T, self.nkv, self.hd)), cos, sin)
        v = v.reshape(T, self.nkv, self.hd)
        if cache is not None:
            if "k" in cache:
                k, v = torch.cat([cache["k"], k]), torch.cat([cache["v"], v])
            cache["k"], cache["v"] = k, v
            L = k.shape[0]
            cu_q = torch.tensor([0, T], dtype=torch.int32, device=x.device)
            cu_k = torch.tensor([0, L], dtype=torch.int32, device=x.device)
            o = ops.attention_varlen(q, k, v, cu_q, cu_k, T, L, causal=True)
        else:
            o = ops.attention_varlen(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=True)
        o = o.reshape(T, -1)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self.o_proj(o)


class SharedExpertMoE(nn.Module):
    """Routed experts plus the always-on shared expert scaled by ``sigmoid(shared_expert_gate(x))``."""

    def __init__(self, c: Qwen35TextConfig, num_local: Optional[int]):
        super().__init__()
        self.routed = SparseMoeBlock(c, num_local)
        f = c.shared_expert_intermediate_size
        self.shared = f > 0
        if self.shared:
            self.shared_gate_up = Linear(c.hidden_size, 2 * f, bias=False)
            self.shared_down = Linear(f, c.hidden_size, bias=False)
            self.shared_expert_gate = Linear(c.hidden_size, 1, bias=False)

    @property
    def aux_loss(self):
        return self.routed.aux_loss

    @property
    def experts(self):
        return self.routed.experts

    def forward(self, x):
        y = self.routed(x)
        if self.shared:
            s = self.shared_down(ops.linear_swiglu(x, self.shared_gate_up.weight))
            y = y + torch.sigmoid(F.linear(x, self.shared_expert_gate.weight)) * s
        return y


class Qwen35DecoderLayer(nn.Module):
    def __init__(self, c: Qwen35TextConfig, linear: bool, num_local: Optional[int] = None):
        super().__init__()
        self.linear = linear
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        if linear:
            self.linear_attn = GatedDeltaNet(c)
        else:
            self.self_attn = GatedAttention(c)
        self.sparse = c.num_experts > 0
        if self.sparse:
            self.mlp = SharedExpertMoE(c, num_local)
        else:
            self.gate_up_proj = Linear(c.hidden_size, 2 * c.intermediate_size, bias=False)
            self.down_proj = Linear(c.intermediate_size, c.hidden_size, bias=False)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen, cache: Optional[dict] = None):
        h = self.input_layernorm(x)
        if self.linear:
            if cache is not None:
                raise NotImplementedError("generation with a recurrent-state cache: decode by prefix re-run (use_cache=False)")
            x = x + self.linear_attn(h, cu_seqlens)
        else:
            x = x + self.self_attn(h, cos, sin, cu_seqlens, max_seqlen, cache)
        h = self.post_attention_layernorm(x)
        if self.sparse:
            return x + self.mlp(h)
        return x + self.down_proj(ops.linear_swiglu(h, self.gate_up_proj.weight))


class MultiTokenPrediction(nn.Module):
    """Multi-token-prediction block (mindspeed_mm/fsdp/models/mtp.py:41-171): for every depth d, the embedding of the
    token one step further and the current hidden state are normalised, concatenated, projected back to the hidden size
    and passed through a full-attention decoder layer; the model's own output head scores the result against the labels
    shifted one more step.  Returns the normalised hidden states of each depth."""

    def __init__(self, c: Qwen35TextConfig, num_local: Optional[int] = None):
        super().__init__()
        self.layers = nn.ModuleList([Qwen35DecoderLayer(c, False, num_local) for _ in range(c.mtp_num_layers)])
        self.pre_fc_norm_embedding = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.pre_fc_norm_hidden = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.fc = Linear(2 * c.hidden_size, c.hidden_size, bias=False)
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps)

    def forward(self, hidden, embeds, depth, cos, sin, cu_seqlens, max_seqlen):
        h = self.fc(torch.cat([self.pre_fc_norm_embedding(embeds), self.pre_fc_norm_hidden(hidden)], dim=-1))
        return self.norm(self.layers[depth](h, cos, sin, cu_seqlens, max_seqlen))


def shift_in_sequences(x: torch.Tensor, cu_seqlens: torch.Tensor, fill) -> torch.Tensor:
    """``out[t] = x[t + 1]`` inside each packed sequence; the last token of every sequence gets ``fill``."""
    out = torch.cat([x[1:], x.new_full((1,), fill)])
    last = cu_seqlens[1:].long() - 1
    out[last[last >= 0]] = fill
    return out


@model_register.register("qwen3_5")
@model_register.register("qwen3_5_moe")
class Qwen35Model(nn.Module):
    """Packed-sequence Qwen3.5 / Qwen3.5-MoE; same batch interface as ``Qwen3VLModel``."""

    def __init__(self, config: Qwen35Config, ep_size: Optional[int] = None):
        super().__init__()
        self.config = config
        t = config.text
        ep = ep_size if ep_size is not None else get_parallel_state().size("ep")
        if t.num_experts and t.num_experts % ep:
            raise ValueError(f"num_experts {t.num_experts} must be divisible by expert_parallel_size {ep}")
        self.visual = Qwen3VisionTransformer(config.vision)
        self.embed_tokens = Embedding(t.vocab_size, t.hidden_size)
        self.layers = nn.ModuleList([Qwen35DecoderLayer(t, t.layer_is_linear(i), t.num_experts // ep if t.num_experts else None)
                                     for i in range(t.num_layers)])
        self.lm_head = LMHead(t)
        self.mtp = MultiTokenPrediction(t, t.num_experts // ep if t.num_experts else None) if t.mtp_num_layers else None
        self.last_mtp_losses = None        # per-depth mean losses of the last forward (detached), for the log
        blocks = [m for m in self.modules() if isinstance(m, SparseMoeBlock)]
        for b in blocks:                    # model-level auxiliary term = coef * mean over MoE layers
            b.aux_scale = t.router_aux_loss_coef / len(blocks)

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                p.copy_(_normal_like(p, self.config.init_std, g))
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)
        for m in self.modules():
            if isinstance(m, GatedDeltaNet):
                m.post_init()

    def fsdp_units(self) -> List[Tuple[str, nn.Module]]:
        v = self.visual
        units = [("embed_tokens", self.embed_tokens), ("visual.patch_embed", v.patch_embed)]
        units += [(f"visual.blocks.{i}", b) for i, b in enumerate(v.blocks)]
        units += [("visual.merger", v.merger)]
        units += [(f"layers.{i}", l) for i, l in enumerate(self.layers)]
        units += [("lm_head", self.lm_head)]
        if self.mtp is not None:
            units += [("mtp", self.mtp)]
        return units

    def expert_units(self):
        out = [(f"layers.{i}.mlp.routed.experts", l.mlp.experts) for i, l in enumerate(self.layers) if l.sparse]
        if self.mtp is not None:
            out += [(f"mtp.layers.{i}.mlp.routed.experts", l.mlp.experts) for i, l in enumerate(self.mtp.layers) if l.sparse]
        return out

    def aux_loss(self):
        """Value of the router load-balancing term of the last forward (detached: its gradient is attached inside the
        MoE blocks, ``models/moe.py: _AttachAux``)."""
        ls = [l.mlp.aux_loss for l in self.layers if l.sparse and l.mlp.aux_loss is not None]
        return self.config.text.router_aux_loss_coef * torch.stack(ls).mean() if ls else None

    def hf_ops(self):
        from ..checkpoint.hf import qwen35_ops
        return qwen35_ops(self.config)

    def forward(self, batch: dict, run=None, kv_cache: Optional[list] = None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        t = self.config.text
        ids = batch["input_ids"]
        x = run(self.embed_tokens, ids)
        pv = batch.get("pixel_values")
        if pv is not None and pv.numel() > 0:
            plan = batch.get("vision_plan") or self.visual.plan(batch["image_grid_thw"], pv.device)
            v, _ = self.visual(pv.to(x.dtype), plan=plan, run=run)
            img_pos = batch.get("image_positions")
            if img_pos is None:
                img_pos = ((ids == self.config.image_token_id) | (ids == self.config.video_token_id)).nonzero(as_tuple=True)[0]
            x = x.index_copy(0, img_pos, v.to(x.dtype))
        cos, sin = batch.get("rope_cos"), batch.get("rope_sin")
        if cos is None:
            rot = int(t.head_dim * t.partial_rotary_factor)
            cos, sin = interleaved_mrope_cos_sin(batch["position_ids"], rot, t.rope_theta, t.mrope_section)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        for i, layer in enumerate(self.layers):
            if kv_cache is not None:
                x = run(layer, x, cos, sin, None, 0, kv_cache[i])
            else:
                x = run(layer, x, cos, sin, batch.get("cu_seqlens"), batch.get("max_seqlen"))
        if kv_cache is not None and batch.get("labels") is None:
            x = x[-1:]
        labels = batch.get("labels")
        if self.mtp is None or labels is None:
            return run(self.lm_head, x, labels)
        loss_sum, n = run(self.lm_head, x, labels)
        # multi-token prediction: depth d predicts the token d + 2 steps ahead from the hidden state of the main stack (after
        # its final norm) and the embedding of the token d + 1 steps ahead; the embedding and the head are the model's own
        cu = batch["cu_seqlens"]
        hidden = run(self.lm_head, x, None, False, True)      # the main stack's final norm lives in the output-head unit
        ids_d, labels_d, extra, self.last_mtp_losses = ids, labels, 0.0, []
        for d in range(t.mtp_num_layers):
            ids_d, labels_d = shift_in_sequences(ids_d, cu, 0), shift_in_sequences(labels_d, cu, -100)
            hidden = run(self.mtp, hidden, run(self.embed_tokens, ids_d), d, cos, sin, cu, batch["max_seqlen"])
            ls, nd = run(self.lm_head, hidden, labels_d, True)
            mean_d = ls / nd.clamp_min(1)
            self.last_mtp_losses.append(mean_d.detach())
            extra = extra + mean_d
        # the caller divides by n: add scaling * mean over depths in the same units
        return loss_sum + (t.mtp_loss_scaling_factor / t.mtp_num_layers) * extra * n, n
