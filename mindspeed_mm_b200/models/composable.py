"""Composable multimodal LM: one implementation, switched by config, behind the zoo's remaining model ids.

The reference keeps one HF-style modeling file per family under ``mindspeed_mm/fsdp/models/*`` and
``mindspeed_mm/models/transformers/*`` (qwen3vl, qwen3omni, glm4v_moe, mistral3, internvl, kimik2_5, kimi_k3, gemma4,
step3_vl, mimov2_5, minimax_m3_vl, longcat_next, qwen3_asr, funasr ...).  Architecturally they are points in one
design space, which this file spans:

* vision tower   : windowed Qwen ViT (``qwen_window``), plain ViT with learned 2-D positions and a 2x2
                   pixel-shuffle MLP projector (``vit``), or none
* audio tower    : windowed Whisper-style encoder, or none
* decoder layers : per-layer token mixer ``attn`` (GQA, optional q/k RMSNorm, optional bias), ``mla`` (low-rank
                   compressed KV with decoupled RoPE), ``gdn`` (gated delta net) or ``kda`` (per-channel gate);
                   per-layer FFN ``dense`` (SwiGLU / GeGLU) or ``moe`` (top-k routed experts + optional shared expert)
* conventions    : Gemma-style ``(1 + w)`` norms and embedding scale, mRoPE or 1-D RoPE

All of them share the packed-sequence batch contract, the FSDP unit plan and the fused loss head of
:class:`~mindspeed_mm_b200.models.qwen2_5_vl.Qwen25VLModel`, so the engine, checkpointing and parallel plans apply
unchanged.  ``PRESETS`` maps the reference's model ids to switch settings (tiny dims for tests; real dims come from
``from_hf_config``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .encoders import WhisperConfig, WhisperEncoder, WhisperLayer
from .qwen2_5_vl import Embedding, Linear, LMHead, Qwen25VLModel, RMSNorm, TextConfig, VisionConfig, VisionTransformer
from .qwen3_5 import GatedDeltaNet, GDNTextConfig
from .moe import MoETextConfig, SparseMoeBlock
from .registry import model_register


# ------------------------------------------------------------------------------------------ config
@dataclass
class DecoderConfig(MoETextConfig, GDNTextConfig):
    mixers: Sequence[str] = ()                 # per layer: attn | mla | gdn | kda   (empty = all attn)
    ffns: Sequence[str] = ()                   # per layer: dense | moe              (empty = all dense)
    shared_expert_intermediate_size: int = 0
    act: str = "silu"                          # silu (SwiGLU) | gelu_tanh (GeGLU)
    norm_plus_one: bool = False                # Gemma: scale by (1 + w)
    embed_scale: bool = False                  # Gemma: embeddings * sqrt(hidden)
    rope: str = "mrope"                        # mrope | rope1d
    qk_norm: bool = False
    # MLA
    kv_lora_rank: int = 64
    q_lora_rank: int = 0
    qk_nope_head_dim: int = 32
    qk_rope_head_dim: int = 16
    v_head_dim: int = 32


@dataclass
class PlainViTConfig:
    patch_size: int = 14
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_layers: int = 24
    num_heads: int = 16
    max_grid: int = 64                          # learned position table is max_grid x max_grid
    merge: int = 2
    out_hidden_size: int = 2048
    in_channels: int = 3
    temporal_patch_size: int = 1
    eps: float = 1e-6


@dataclass
class ComposableConfig:
    text: DecoderConfig = field(default_factory=DecoderConfig)
    vision_kind: Optional[str] = "qwen_window"  # qwen_window | vit | None
    vision: Optional[VisionConfig] = None
    vit: Optional[PlainViTConfig] = None
    audio: Optional[WhisperConfig] = None
    audio_window: int = 100
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    audio_token_id: int = 151646
    init_std: float = 0.02
    tile_format: bool = False                   # any-resolution tiles: line-break and view-separator embeddings
    global_view_pos: str = "head"               # head | tail: where the global view sits relative to the local grid


# ------------------------------------------------------------------------------------------ blocks
class ScaledRMSNorm(RMSNorm):
    """Gemma convention: the stored weight is an offset from one."""

    def forward(self, x):
        return ops.rms_norm(x, self.weight + 1.0, self.eps)


def _norm(c: DecoderConfig, dim: int):
    return ScaledRMSNorm(dim, c.rms_norm_eps) if c.norm_plus_one else RMSNorm(dim, c.rms_norm_eps)


class GQAttention(nn.Module):
    def __init__(self, c: DecoderConfig):
        super().__init__()
        self.nq, self.nkv, self.hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        self.qkv_proj = Linear(c.hidden_size, (self.nq + 2 * self.nkv) * self.hd, bias=c.qkv_bias)
        self.o_proj = Linear(self.nq * self.hd, c.hidden_size, bias=False)
        self.q_norm = _norm(c, self.hd) if c.qk_norm else None
        self.k_norm = _norm(c, self.hd) if c.qk_norm else None

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        T = x.shape[0]
        q, k, v = self.qkv_proj(x).split([self.nq * self.hd, self.nkv * self.hd, self.nkv * self.hd], dim=-1)
        q, k = q.reshape(T, self.nq, self.hd), k.reshape(T, self.nkv, self.hd)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = ops.rope_rotate_half(q, cos, sin), ops.rope_rotate_half(k, cos, sin)
        o = ops.attention_varlen(q, k, v.reshape(T, self.nkv, self.hd), cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                 causal=True)
        return self.o_proj(o.reshape(T, -1))


class MLAttention(nn.Module):
    """Multi-head latent attention: K/V are expanded from a shared low-rank latent; RoPE acts on a separate
    ``qk_rope_head_dim`` slice whose key part is shared by all heads (DeepSeek-V2/V3 and the Kimi-K2 family)."""

    def __init__(self, c: DecoderConfig):
        super().__init__()
        self.n = c.num_attention_heads
        self.dn, self.dr, self.dv, self.r = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank
        dq = self.n * (self.dn + self.dr)
        if c.q_lora_rank:
            self.q_a_proj = Linear(c.hidden_size, c.q_lora_rank, bias=False)
            self.q_a_norm = _norm(c, c.q_lora_rank)
            self.q_b_proj = Linear(c.q_lora_rank, dq, bias=False)
        else:
            self.q_proj = Linear(c.hidden_size, dq, bias=False)
        self.kv_a_proj = Linear(c.hidden_size, self.r + self.dr, bias=False)
        self.kv_a_norm = _norm(c, self.r)
        self.kv_b_proj = Linear(self.r, self.n * (self.dn + self.dv), bias=False)
        self.o_proj = Linear(self.n * self.dv, c.hidden_size, bias=False)
        self.scale = (self.dn + self.dr) ** -0.5

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        T = x.shape[0]
        q = self.q_b_proj(self.q_a_norm(self.q_a_proj(x))) if hasattr(self, "q_a_proj") else self.q_proj(x)
        q = q.view(T, self.n, self.dn + self.dr)
        kv_a = self.kv_a_proj(x)
        latent, k_rope = kv_a[:, : self.r], kv_a[:, self.r:]
        kv = self.kv_b_proj(self.kv_a_norm(latent)).view(T, self.n, self.dn + self.dv)
        cr, sr = cos[..., : self.dr], sin[..., : self.dr]
        q_rope = ops.rope_rotate_half(q[..., self.dn:].contiguous(), cr, sr)
        k_rope = ops.rope_rotate_half(k_rope.reshape(T, 1, self.dr).contiguous(), cr, sr).expand(T, self.n, self.dr)
        qf = torch.cat([q[..., : self.dn], q_rope], dim=-1)
        kf = torch.cat([kv[..., : self.dn], k_rope], dim=-1)
        d = self.dn + self.dr
        v = kv[..., self.dn:]
        if self.dv < d:                                   # one head size for the attention kernel: zero-pad V
            v = F.pad(v, (0, d - self.dv))
        o = ops.attention_varlen(qf.contiguous(), kf.contiguous(), v.contiguous(), cu_seqlens, cu_seqlens, max_seqlen,
                                 max_seqlen, causal=True, softmax_scale=self.scale)
        return self.o_proj(o[..., : self.dv].reshape(T, self.n * self.dv))


class KimiDeltaAttention(nn.Module):
    """Delta-rule mixer with a per-channel forget gate (``ops.kda``); projections follow the GDN block."""

    def __init__(self, c: DecoderConfig):
        super().__init__()
        self.h, self.dk, self.dv = c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim
        self.q_proj = Linear(c.hidden_size, self.h * self.dk, bias=False)
        self.k_proj = Linear(c.hidden_size, self.h * self.dk, bias=False)
        self.v_proj = Linear(c.hidden_size, self.h * self.dv, bias=False)
        self.g_proj = Linear(c.hidden_size, self.h * self.dk, bias=False)
        self.b_proj = Linear(c.hidden_size, self.h, bias=False)
        self.o_proj = Linear(self.h * self.dv, c.hidden_size, bias=False)
        self.chunk = c.gdn_chunk

    def forward(self, x, cu_seqlens):
        T = x.shape[0]
        q = ops.l2_norm(F.silu(self.q_proj(x)).view(T, self.h, self.dk))
        k = ops.l2_norm(F.silu(self.k_proj(x)).view(T, self.h, self.dk))
        v = F.silu(self.v_proj(x)).view(T, self.h, self.dv)
        g = -F.softplus(self.g_proj(x).float()).view(T, self.h, self.dk)
        beta = torch.sigmoid(self.b_proj(x).float())
        if self.chunk == 64:
            o = ops.kda_varlen(q, k, v, g, beta, cu_seqlens)
        else:
            outs = []
            cu = cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
            for a, b in zip(cu[:-1], cu[1:]):
                o, _ = ops.kda(q[None, a:b], k[None, a:b], v[None, a:b], g[None, a:b], beta[None, a:b], chunk=self.chunk)
                outs.append(o[0])
            o = torch.cat(outs, 0)
        return self.o_proj(o.to(x.dtype).reshape(T, self.h * self.dv))


class GatedMLP(nn.Module):
    def __init__(self, hidden, inter, act):
        super().__init__()
        self.act = act
        self.gate_up_proj = Linear(hidden, 2 * inter, bias=False)
        self.down_proj = Linear(inter, hidden, bias=False)

    def forward(self, x):
        if self.act == "silu":
            return self.down_proj(ops.linear_swiglu(x, self.gate_up_proj.weight))
        g, u = self.gate_up_proj(x).chunk(2, dim=-1)
        return self.down_proj(ops.gelu_tanh(g) * u)


class MoEWithShared(nn.Module):
    def __init__(self, c: DecoderConfig, num_local: Optional[int]):
        super().__init__()
        self.routed = SparseMoeBlock(c, num_local)
        self.shared = GatedMLP(c.hidden_size, c.shared_expert_intermediate_size, c.act) \
            if c.shared_expert_intermediate_size else None

    @property
    def aux_loss(self):
        return self.routed.aux_loss

    def forward(self, x):
        y = self.routed(x)
        return y + self.shared(x) if self.shared is not None else y


class ComposableLayer(nn.Module):
    def __init__(self, c: DecoderConfig, mixer: str, ffn: str, num_local_experts: Optional[int] = None):
        super().__init__()
        self.kind = mixer
        self.input_layernorm = _norm(c, c.hidden_size)
        self.post_attention_layernorm = _norm(c, c.hidden_size)
        self.mixer = {"attn": GQAttention, "mla": MLAttention, "gdn": GatedDeltaNet, "kda": KimiDeltaAttention}[mixer](c)
        self.mlp = MoEWithShared(c, num_local_experts) if ffn == "moe" else GatedMLP(c.hidden_size, c.intermediate_size, c.act)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        h = self.input_layernorm(x)
        if self.kind in ("gdn", "kda"):
            x = x + self.mixer(h, cu_seqlens)
        else:
            x = x + self.mixer(h, cos, sin, cu_seqlens, max_seqlen)
        return x + self.mlp(self.post_attention_layernorm(x))


# ------------------------------------------------------------------------------------------ towers
class ViTBlock(nn.Module):
    def __init__(self, c: PlainViTConfig):
        super().__init__()
        self.heads = c.num_heads
        self.ln1 = ops.LayerNorm(c.hidden_size, eps=c.eps)
        self.qkv = Linear(c.hidden_size, 3 * c.hidden_size, bias=True)
        self.proj = Linear(c.hidden_size, c.hidden_size, bias=True)
        self.ln2 = ops.LayerNorm(c.hidden_size, eps=c.eps)
        self.fc1 = Linear(c.hidden_size, c.intermediate_size, bias=True)
        self.fc2 = Linear(c.intermediate_size, c.hidden_size, bias=True)

    def forward(self, x, cu_seqlens, max_seqlen):
        T, H = x.shape
        qkv = self.qkv(self.ln1(x)).view(T, 3, self.heads, H // self.heads)
        o = ops.attention_varlen(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=False)
        x = x + self.proj(o.reshape(T, H))
        return x + self.fc2(ops.gelu_tanh(self.fc1(self.ln2(x))))


class PlainViT(nn.Module):
    """ViT over flattened patch rows in 2x2-merge order (the collator's layout); per-image full attention; the
    projector concatenates each merge x merge group (a pixel shuffle) and maps it to the LLM width."""

    def __init__(self, c: PlainViTConfig):
        super().__init__()
        self.cfg = c
        self.patch_embed = Linear(c.in_channels * c.temporal_patch_size * c.patch_size ** 2, c.hidden_size, bias=True)
        self.pos_embed = nn.Parameter(torch.empty(c.max_grid * c.max_grid, c.hidden_size))
        self.blocks = nn.ModuleList(ViTBlock(c) for _ in range(c.num_layers))
        self.merger = nn.Sequential()
        m2 = c.merge ** 2
        self.merger_norm = ops.LayerNorm(c.hidden_size * m2, eps=c.eps)
        self.merger_fc1 = Linear(c.hidden_size * m2, c.out_hidden_size, bias=True)
        self.merger_fc2 = Linear(c.out_hidden_size, c.out_hidden_size, bias=True)

    def position_index(self, grid_thw: torch.Tensor) -> torch.Tensor:
        m, idx = self.cfg.merge, []
        for t, h, w in grid_thw.tolist():
            r = torch.arange(h).view(h // m, m, 1, 1).expand(h // m, m, w // m, m).permute(0, 2, 1, 3)
            c = torch.arange(w).view(1, 1, w // m, m).expand(h // m, m, w // m, m).permute(0, 2, 1, 3)
            idx.append((r * self.cfg.max_grid + c).reshape(-1).repeat(t))
        return torch.cat(idx)

    def forward(self, pixel_values, grid_thw):
        x = self.patch_embed(pixel_values)
        x = x + self.pos_embed[self.position_index(grid_thw).to(x.device)].to(x.dtype)
        lens = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])
        cu = F.pad(lens.cumsum(0), (1, 0)).to(device=x.device, dtype=torch.int32)
        mx = int(lens.max())
        for blk in self.blocks:
            x = blk(x, cu, mx)
        x = self.merger_norm(x.view(-1, x.shape[-1] * self.cfg.merge ** 2))
        return self.merger_fc2(ops.gelu(self.merger_fc1(x)))


class TileFormatter(nn.Module):
    """Lays the per-view features of any-resolution images out as the prompt expects them: the global view row by row
    with a learned line-break vector after every row, a learned separator, then the local views stitched into one
    ``(tiles_h * h) x (tiles_w * w)`` map, again with a line break per row (reference:
    mindspeed_mm/models/deepseekvl_model.py:313-428, ``tile_tag == "2D"``).  ``data/anyres.py`` emits the placeholder
    tokens in the same order."""

    def __init__(self, dim: int, global_view_pos: str = "head"):
        super().__init__()
        self.image_newline = nn.Parameter(torch.empty(dim))
        self.view_separator = nn.Parameter(torch.empty(dim))
        self.global_view_pos = global_view_pos

    def forward(self, feats, spatial_crop):
        """feats [n_views * h * w, D] (views of all images in order: global, then local row-major);
        spatial_crop [n_images, 2] = (tiles_w, tiles_h).  -> [sum of image_token_count, D]."""
        crops = spatial_crop.tolist()
        n_views = sum(1 + tw * th for tw, th in crops)
        D = feats.shape[-1]
        hw = feats.shape[0] // max(n_views, 1)
        h = w = int(round(hw ** 0.5))
        f = feats.view(n_views, h, w, D)
        nl = self.image_newline.to(feats.dtype)
        sep = self.view_separator.to(feats.dtype)[None]
        out, at = [], 0
        for tw, th in crops:
            g = torch.cat([f[at], nl.expand(h, 1, D)], 1).reshape(-1, D)
            loc = f[at + 1: at + 1 + tw * th].view(th, tw, h, w, D).permute(0, 2, 1, 3, 4).reshape(th * h, tw * w, D)
            loc = torch.cat([loc, nl.expand(th * h, 1, D)], 1).reshape(-1, D)
            out += [g, sep, loc] if self.global_view_pos == "head" else [loc, sep, g]
            at += 1 + tw * th
        return torch.cat(out)


class AudioTower(nn.Module):
    def __init__(self, c: WhisperConfig, window: int, out_dim: int):
        super().__init__()
        from .encoders import WindowedAudioEncoder
        self.tower = WindowedAudioEncoder(c, window, out_dim)

    def forward(self, mels):
        return torch.cat(self.tower(mels), 0)


# ------------------------------------------------------------------------------------------ model
@model_register.register("composable_lm")
class ComposableLM(Qwen25VLModel):
    def __init__(self, config: ComposableConfig, ep_size: int = 1):
        nn.Module.__init__(self)
        self.config = config
        t = config.text
        mixers = list(t.mixers) or ["attn"] * t.num_layers
        ffns = list(t.ffns) or ["dense"] * t.num_layers
        if len(mixers) != t.num_layers or len(ffns) != t.num_layers:
            raise ValueError("mixers / ffns must list one entry per layer")
        self.visual = None
        if config.vision_kind == "qwen_window":
            self.visual = VisionTransformer(config.vision)
        elif config.vision_kind == "vit":
            self.visual = PlainViT(config.vit)
        self.audio = AudioTower(config.audio, config.audio_window, t.hidden_size) if config.audio is not None else None
        self.tile_format = TileFormatter(t.hidden_size, config.global_view_pos) if config.tile_format else None
        self.embed_tokens = Embedding(t.vocab_size, t.hidden_size)
        self.layers = nn.ModuleList(ComposableLayer(t, m, f, t.num_experts // ep_size if f == "moe" else None)
                                    for m, f in zip(mixers, ffns))
        self.lm_head = LMHead(t)
        if t.norm_plus_one:
            self.lm_head.norm = _norm(t, t.hidden_size)
        self._set_aux_scale()

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        super().init_weights(seed)
        for m in self.modules():
            if isinstance(m, GatedDeltaNet):
                m.post_init()
            if isinstance(m, ScaledRMSNorm):
                m.weight.zero_()
            if isinstance(m, TileFormatter):
                g = torch.Generator(device="cpu").manual_seed(seed + 17)
                for p in (m.image_newline, m.view_separator):
                    p.copy_(torch.randn(p.shape, generator=g) * self.config.init_std)

    def fsdp_units(self) -> List[Tuple[str, nn.Module]]:
        units: List[Tuple[str, nn.Module]] = [("embed_tokens", self.embed_tokens)]
        if isinstance(self.visual, VisionTransformer):
            units += [("visual.patch_embed", self.visual.patch_embed)]
            units += [(f"visual.blocks.{i}", b) for i, b in enumerate(self.visual.blocks)]
            units += [("visual.merger", self.visual.merger)]
        elif self.visual is not None:
            units += [("visual", self.visual)]
        if self.tile_format is not None:
            units += [("tile_format", self.tile_format)]
        if self.audio is not None:
            units += [("audio", self.audio)]
        units += [(f"layers.{i}", l) for i, l in enumerate(self.layers)]
        return units + [("lm_head", self.lm_head)]

    def expert_units(self):
        return [(f"layers.{i}.mlp.routed.experts", l.mlp.routed.experts) for i, l in enumerate(self.layers)
                if isinstance(l.mlp, MoEWithShared)]

    def _set_aux_scale(self):
        blocks = [m for m in self.modules() if isinstance(m, SparseMoeBlock)]
        for b in blocks:                    # model-level auxiliary term = coef * mean over MoE layers
            b.aux_scale = self.config.text.router_aux_loss_coef / len(blocks)

    def aux_loss(self):
        """Value of the router load-balancing term of the last forward (detached; the gradient is attached inside the
        MoE blocks)."""
        t = self.config.text
        ls = [l.mlp.aux_loss for l in self.layers if isinstance(l.mlp, MoEWithShared) and l.mlp.aux_loss is not None]
        return t.router_aux_loss_coef * torch.stack(ls).mean() if ls else None

    def forward(self, batch: dict, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        cfg, t = self.config, self.config.text
        ids = batch.get("input_ids")
        x = batch.get("inputs_embeds")            # callers that build their own token embeddings (speech LMs)
        if x is None:
            x = run(self.embed_tokens, ids)
            if t.embed_scale:
                x = x * math.sqrt(t.hidden_size)
        pv = batch.get("pixel_values")
        if self.visual is not None and pv is not None and pv.numel() > 0:
            if isinstance(self.visual, VisionTransformer):
                vis = self.visual
                plan = batch.get("vision_plan") or vis.plan(batch["image_grid_thw"], pv.device)
                v = run(vis.patch_embed, pv.to(x.dtype)).index_select(0, plan["perm"])
                for i in range(len(vis.blocks)):
                    full = i in vis.cfg.fullatt_block_indexes
                    cu, mx = (plan["cu_full"], plan["max_full"]) if full else (plan["cu_win"], plan["max_win"])
                    v = run(vis.blocks[i], v, plan["cos"].to(x.dtype), plan["sin"].to(x.dtype), cu, mx)
                v = run(vis.merger, v).index_select(0, plan["reverse"])
            else:
                v = run(self.visual, pv.to(x.dtype), batch["image_grid_thw"])
            if self.tile_format is not None and batch.get("spatial_crop") is not None:
                v = run(self.tile_format, v, batch["spatial_crop"])
            pos = batch.get("image_positions")
            if pos is None:
                pos = (ids == cfg.image_token_id).nonzero(as_tuple=True)[0]
            x = x.index_copy(0, pos, v.to(x.dtype))
        mels = batch.get("audio_features")
        if self.audio is not None and mels:
            a = run(self.audio, [m.to(x.dtype) for m in mels])
            pos = (ids == cfg.audio_token_id).nonzero(as_tuple=True)[0]
            x = x.index_copy(0, pos, a[: pos.numel()].to(x.dtype))
        pos_ids = batch["position_ids"]
        rope_dim = t.qk_rope_head_dim if "mla" in (t.mixers or ()) and "attn" not in (t.mixers or ()) else t.head_dim
        if t.rope == "mrope":
            cos, sin = ops.ref.mrope_cos_sin(pos_ids, rope_dim, t.rope_theta, t.mrope_section)
        else:
            p1 = pos_ids[0] if pos_ids.dim() == 2 else pos_ids
            cos, sin = ops.ref.mrope_cos_sin(p1[None].expand(3, -1), rope_dim, t.rope_theta, (rope_dim // 2, 0, 0))
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        trace = batch.get("collect_hidden")       # a list: receives the embeddings and every layer's output
        if trace is not None:
            trace.append(x)
        for layer in self.layers:
            x = run(layer, x, cos, sin, batch["cu_seqlens"], batch["max_seqlen"])
            if trace is not None:
                trace.append(x)
        if batch.get("return_hidden"):
            return x                              # pre-norm hidden states [T, H]
        return run(self.lm_head, x, batch.get("labels"))


    def hidden_states(self, batch: dict, run=None) -> List[torch.Tensor]:
        """Embeddings followed by the output of every layer (pre final norm), each [T, H]: what prompt encoders that read
        an inner layer of a language model need."""
        trace: List[torch.Tensor] = []
        self.forward({**batch, "collect_hidden": trace, "return_hidden": True}, run=run)
        return trace

    def final_norm(self, h):
        return self.lm_head.norm(h)


# ------------------------------------------------------------------------------------------ presets
def _tiny_text(**kw) -> DecoderConfig:
    base = dict(num_layers=2, hidden_size=128, intermediate_size=256, num_attention_heads=4, num_key_value_heads=2,
                head_dim=32, vocab_size=1024, qkv_bias=False, mrope_section=(4, 6, 6), num_experts=4, num_experts_per_tok=2,
                moe_intermediate_size=64, linear_num_key_heads=2, linear_num_value_heads=2, linear_key_head_dim=32,
                linear_value_head_dim=32, gdn_chunk=16)
    return DecoderConfig(**{**base, **kw})


def _tiny_qwen_vit(out):
    return VisionConfig(depth=1, hidden_size=64, intermediate_size=128, num_heads=2, fullatt_block_indexes=(0,), out_hidden_size=out)


def _tiny_vit(out):
    return PlainViTConfig(hidden_size=64, intermediate_size=128, num_layers=1, num_heads=2, max_grid=16, out_hidden_size=out)


def _tiny_audio():
    return WhisperConfig.tiny()


_IDS = dict(image_token_id=1023, video_token_id=1022, vision_start_token_id=1021, audio_token_id=1020)

# model id (as the reference registers it) -> tiny configuration exercising that family's switches
PRESETS: Dict[str, ComposableConfig] = {
    "qwen2vl": ComposableConfig(_tiny_text(qkv_bias=True), "qwen_window", _tiny_qwen_vit(128), **_IDS),
    "qwen3omni": ComposableConfig(_tiny_text(qk_norm=True, ffns=("moe", "moe")), "qwen_window", _tiny_qwen_vit(128),
                                  audio=_tiny_audio(), audio_window=20, **_IDS),
    "qwen3_asr": ComposableConfig(_tiny_text(qk_norm=True, rope="rope1d"), None, audio=_tiny_audio(), audio_window=20, **_IDS),
    "funasr": ComposableConfig(_tiny_text(rope="rope1d"), None, audio=_tiny_audio(), audio_window=20, **_IDS),
    "glm4v_moe": ComposableConfig(_tiny_text(qkv_bias=True, ffns=("dense", "moe"), shared_expert_intermediate_size=64),
                                  "qwen_window", _tiny_qwen_vit(128), **_IDS),
    "mistral3": ComposableConfig(_tiny_text(rope="rope1d"), "vit", vit=_tiny_vit(128), **_IDS),
    "gemma4": ComposableConfig(_tiny_text(rope="rope1d", act="gelu_tanh", norm_plus_one=True, embed_scale=True, qk_norm=True),
                               "vit", vit=_tiny_vit(128), **_IDS),
    "step3_vl": ComposableConfig(_tiny_text(rope="rope1d", ffns=("dense", "moe"), shared_expert_intermediate_size=64),
                                 "vit", vit=_tiny_vit(128), **_IDS),
    "kimik2_5": ComposableConfig(_tiny_text(rope="rope1d", mixers=("mla", "mla"), ffns=("dense", "moe"),
                                            shared_expert_intermediate_size=64, q_lora_rank=48), "vit", vit=_tiny_vit(128), **_IDS),
    "kimi_k3": ComposableConfig(_tiny_text(rope="rope1d", mixers=("kda", "mla"), ffns=("moe", "moe"),
                                           shared_expert_intermediate_size=64), "vit", vit=_tiny_vit(128), **_IDS),
    "mimov2_5": ComposableConfig(_tiny_text(qk_norm=True, ffns=("moe", "moe")), "qwen_window", _tiny_qwen_vit(128), **_IDS),
    "minimax_m3_vl": ComposableConfig(_tiny_text(qk_norm=True, rope="rope1d", ffns=("moe", "moe")), "vit", vit=_tiny_vit(128), **_IDS),
    # Chameleon-style autoregressive image generation: image patches are MOVQ code indices inside the text vocabulary
    "lumina_mgpt2": ComposableConfig(_tiny_text(qk_norm=True, rope="rope1d"), None, **_IDS),
    # LLaVA-style assembly (plain ViT + projector + dense decoder) and DeepSeek-VL2 (plain ViT + MLA attention + routed experts)
    "llava": ComposableConfig(_tiny_text(rope="rope1d"), "vit", vit=_tiny_vit(128), **_IDS),
    "deepseekvl2": ComposableConfig(_tiny_text(rope="rope1d", mixers=("mla", "mla"), ffns=("dense", "moe"),
                                               shared_expert_intermediate_size=64), "vit", vit=_tiny_vit(128), tile_format=True, **_IDS),
    "longcat_next": ComposableConfig(_tiny_text(rope="rope1d", mixers=("mla", "mla"), ffns=("moe", "moe")), "vit",
                                     vit=_tiny_vit(128), **_IDS),
}


def build_preset(model_id: str, **text_overrides) -> ComposableLM:
    cfg = PRESETS[model_id]
    if text_overrides:
        cfg = replace(cfg, text=replace(cfg.text, **text_overrides))
    return ComposableLM(cfg)


def _preset_factory(mid: str):
    def build(config=None, **kw):
        return ComposableLM(config if isinstance(config, ComposableConfig) else PRESETS[mid], **kw)
    # a family id without its own modeling file: with a Hugging Face checkpoint directory the trainer builds the stock
    # transformers class instead (plugins/hf_auto.py), so real dimensions and published weights load by name
    build.hf_fallback = True
    build.__name__ = f"composable_{mid}"
    return build


for _mid in PRESETS:
    model_register.register(_mid)(_preset_factory(_mid))


def from_hf_config(hf: dict) -> ComposableConfig:
    """Map a HuggingFace ``config.json`` (text_config / vision_config blocks) onto the switches above."""
    tc = hf.get("text_config", hf)
    n = tc["num_hidden_layers"]
    moe = tc.get("num_experts") or tc.get("n_routed_experts") or 0
    dense_first = tc.get("first_k_dense_replace", 0)
    step = tc.get("decoder_sparse_step", 1) or 1
    ffns = tuple("moe" if moe and i >= dense_first and (i + 1) % step == 0 else "dense" for i in range(n))
    mla = "kv_lora_rank" in tc
    types = tc.get("layer_types")
    if types:
        mixers = tuple("gdn" if "linear" in ty else ("mla" if mla else "attn") for ty in types)
    else:
        mixers = tuple(["mla" if mla else "attn"] * n)
    heads = tc["num_attention_heads"]
    text = DecoderConfig(
        num_layers=n, hidden_size=tc["hidden_size"], intermediate_size=tc.get("intermediate_size", 4 * tc["hidden_size"]),
        num_attention_heads=heads, num_key_value_heads=tc.get("num_key_value_heads", heads),
        head_dim=tc.get("head_dim", tc["hidden_size"] // heads), vocab_size=tc["vocab_size"],
        qkv_bias=tc.get("attention_bias", tc.get("qkv_bias", False)), rms_norm_eps=tc.get("rms_norm_eps", 1e-6),
        rope_theta=tc.get("rope_theta", 1e6),
        mrope_section=tuple((tc.get("rope_scaling") or {}).get("mrope_section", (16, 24, 24))),
        rope="mrope" if (tc.get("rope_scaling") or {}).get("mrope_section") else "rope1d",
        num_experts=moe or 1, num_experts_per_tok=tc.get("num_experts_per_tok", 1),
        moe_intermediate_size=tc.get("moe_intermediate_size", tc.get("intermediate_size", 0)),
        shared_expert_intermediate_size=tc.get("shared_expert_intermediate_size", 0) or
        tc.get("n_shared_experts", 0) * tc.get("moe_intermediate_size", 0),
        qk_norm=tc.get("use_qk_norm", "qwen3" in hf.get("model_type", "")), mixers=mixers, ffns=ffns,
        kv_lora_rank=tc.get("kv_lora_rank", 64), q_lora_rank=tc.get("q_lora_rank") or 0,
        qk_nope_head_dim=tc.get("qk_nope_head_dim", 32), qk_rope_head_dim=tc.get("qk_rope_head_dim", 16),
        v_head_dim=tc.get("v_head_dim", 32), act="gelu_tanh" if "gelu" in tc.get("hidden_act", "silu") else "silu",
        norm_plus_one="gemma" in hf.get("model_type", ""), embed_scale="gemma" in hf.get("model_type", ""))
    vc = hf.get("vision_config")
    kind, vision, vit = None, None, None
    if vc:
        if "window_size" in vc or "fullatt_block_indexes" in vc or "spatial_merge_size" in vc:
            kind = "qwen_window"
            depth = vc.get("depth", vc.get("num_hidden_layers", 32))
            vision = VisionConfig(depth=depth, hidden_size=vc["hidden_size"], intermediate_size=vc["intermediate_size"],
                                  num_heads=vc["num_heads"], patch_size=vc.get("patch_size", 14),
                                  window_size=vc.get("window_size", 112),
                                  fullatt_block_indexes=tuple(vc.get("fullatt_block_indexes", range(depth))),
                                  out_hidden_size=vc.get("out_hidden_size", text.hidden_size))
        else:
            kind = "vit"
            vit = PlainViTConfig(patch_size=vc.get("patch_size", 14), hidden_size=vc["hidden_size"],
                                 intermediate_size=vc["intermediate_size"], num_layers=vc["num_hidden_layers"],
                                 num_heads=vc["num_attention_heads"], out_hidden_size=text.hidden_size)
    return ComposableConfig(text=text, vision_kind=kind, vision=vision, vit=vit,
                            image_token_id=hf.get("image_token_id", 151655), video_token_id=hf.get("video_token_id", 151656),
                            vision_start_token_id=hf.get("vision_start_token_id", 151652))
