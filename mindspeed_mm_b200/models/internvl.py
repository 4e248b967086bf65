"""InternVL3 / InternVL3.5: InternViT tiles -> pixel-shuffle projector -> Qwen2 / Qwen3 decoder with 1-D RoPE.

Reference: mindspeed_mm/fsdp/models/internvl (InternVL3.5 chat model on the transformers-backed trainer) and the Hugging
Face ``internvl`` modeling whose checkpoints it loads.  What sets the family apart from the Qwen-VL towers:

* vision: every image is cut into 448 x 448 tiles (``data/anyres.py`` picks the tile grid); a tile is one sequence of
  ``1 + (448 / 14)^2`` tokens (class token first) with a learned absolute position table, bicubically resized when the
  tile size differs from the table's; blocks are pre-norm (LayerNorm, or RMSNorm on the 6B tower) with a learned
  per-channel scale on both residual branches (``lambda_1`` / ``lambda_2``); the 6B tower also RMS-normalises q and k
  over the WHOLE embedding width before the head split
* connector: drop the class token, regroup 2 x 2 neighbouring patches into the channel dim (the published "pixel
  shuffle" order: row pairs first, then column pairs, then a transpose back), LayerNorm -> Linear -> GELU -> Linear
* text: a plain Qwen2 (QKV bias), Qwen3 (per-head q/k RMSNorm) or Qwen3-MoE (routed experts) decoder; positions restart in every packed sequence

Packed-sequence training interface shared by the VLMs: ``forward(batch, run)`` -> ``(loss_sum, n_valid)`` or logits.
``batch["pixel_values"]`` is ``[n_tiles, 3, H, W]``; the tiles' tokens replace the image placeholder tokens in order.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..parallel.state import get_parallel_state
from .moe import MoETextConfig, SparseMoeBlock
from .qwen2_5_vl import Embedding, Linear, LMHead, RMSNorm, _normal_like
from .qwen3_vl import Qwen3DecoderLayer
from .registry import model_register


@dataclass
class InternViTConfig:
    depth: int = 24
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_heads: int = 16
    image_size: int = 448
    patch_size: int = 14
    in_channels: int = 3
    norm_type: str = "layer_norm"           # "rms_norm" on InternViT-6B
    use_qk_norm: bool = False               # InternViT-6B
    attention_bias: bool = True
    eps: float = 1e-6
    layer_scale_init: float = 0.1
    final_layernorm: bool = False           # HF ``use_mean_pooling = False`` keeps a LayerNorm after the last block


@dataclass
class InternVLTextConfig(MoETextConfig):
    num_experts: int = 0
    qk_norm: bool = True                    # Qwen3 decoder (InternVL3.5); False + qkv_bias = Qwen2 (InternVL3)
    qkv_bias: bool = False
    rope_theta: float = 1e6


@dataclass
class InternVLConfig:
    vision: InternViTConfig = field(default_factory=InternViTConfig)
    text: InternVLTextConfig = field(default_factory=InternVLTextConfig)
    downsample_ratio: float = 0.5
    image_token_id: int = 151671            # <IMG_CONTEXT>; <img> and </img> sit just before it in the vocabulary
    vision_start_token_id: Optional[int] = None
    vision_end_token_id: Optional[int] = None
    init_std: float = 0.02

    def __post_init__(self):
        if self.vision_start_token_id is None:
            self.vision_start_token_id = self.image_token_id - 2
        if self.vision_end_token_id is None:
            self.vision_end_token_id = self.image_token_id - 1

    @property
    def tokens_per_tile(self) -> int:
        side = self.vision.image_size // self.vision.patch_size
        return int(side * self.downsample_ratio) ** 2

    @staticmethod
    def internvl3_5_8b():
        """InternVL3.5-8B: InternViT-300M + Qwen3-8B."""
        return InternVLConfig(text=InternVLTextConfig(
            num_layers=36, hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8,
            head_dim=128, vocab_size=151936))

    @staticmethod
    def internvl3_5_30b_a3b():
        """InternVL3.5-30B-A3B: InternViT-300M + Qwen3-30B-A3B (128 routed experts, 8 per token)."""
        return InternVLConfig(text=InternVLTextConfig(
            num_layers=48, hidden_size=2048, intermediate_size=6144, num_attention_heads=32, num_key_value_heads=4,
            head_dim=128, vocab_size=151936, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768))

    @staticmethod
    def internvl3_8b():
        """InternVL3-8B: InternViT-300M + Qwen2.5-7B."""
        return InternVLConfig(image_token_id=151667, text=InternVLTextConfig(
            num_layers=28, hidden_size=3584, intermediate_size=18944, num_attention_heads=28, num_key_value_heads=4,
            vocab_size=151674, qk_norm=False, qkv_bias=True))

    @staticmethod
    def internvl3_5_38b():
        """InternVL3.5-38B: InternViT-6B (RMSNorm, q/k norm) + Qwen3-32B."""
        return InternVLConfig(
            vision=InternViTConfig(depth=45, hidden_size=3200, intermediate_size=12800, num_heads=25,
                                   norm_type="rms_norm", use_qk_norm=True, attention_bias=False),
            text=InternVLTextConfig(num_layers=64, hidden_size=5120, intermediate_size=25600, num_attention_heads=64,
                                    num_key_value_heads=8, head_dim=128, vocab_size=151936))

    @staticmethod
    def tiny(qwen3: bool = True, big_tower: bool = False, moe: bool = False):
        v = InternViTConfig(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, image_size=56, patch_size=14,
                            norm_type="rms_norm" if big_tower else "layer_norm", use_qk_norm=big_tower,
                            attention_bias=not big_tower, final_layernorm=big_tower)
        t = InternVLTextConfig(num_layers=2, hidden_size=64, intermediate_size=128, num_attention_heads=4,
                               num_key_value_heads=2, head_dim=16, vocab_size=160, qk_norm=qwen3, qkv_bias=not qwen3)
        if moe:
            t.num_experts, t.num_experts_per_tok, t.moe_intermediate_size, t.router_aux_loss_coef = 8, 2, 32, 0.001
        return InternVLConfig(vision=v, text=t, image_token_id=150)

    @staticmethod
    def from_hf(hf: dict) -> "InternVLConfig":
        """From a Hugging Face ``config.json`` (``model_type: internvl``)."""
        vc, tc = hf.get("vision_config", {}), hf.get("text_config", {})

        def one(x):
            return x[0] if isinstance(x, (list, tuple)) else x

        v = InternViTConfig(
            depth=vc.get("num_hidden_layers", 24), hidden_size=vc.get("hidden_size", 1024),
            intermediate_size=vc.get("intermediate_size", 4096), num_heads=vc.get("num_attention_heads", 16),
            image_size=one(vc.get("image_size", 448)), patch_size=one(vc.get("patch_size", 14)),
            norm_type=vc.get("norm_type", "layer_norm"), use_qk_norm=vc.get("use_qk_norm", False),
            attention_bias=vc.get("attention_bias", False), eps=vc.get("layer_norm_eps", 1e-6),
            layer_scale_init=vc.get("layer_scale_init_value", 0.1),
            final_layernorm=not vc.get("use_mean_pooling", True))
        qwen3 = tc.get("model_type", "qwen2") in ("qwen3", "qwen3_moe")
        moe = dict(num_experts=tc.get("num_experts", tc.get("num_local_experts", 0)), num_experts_per_tok=tc.get("num_experts_per_tok", 8),
                   moe_intermediate_size=tc.get("moe_intermediate_size", 768), norm_topk_prob=tc.get("norm_topk_prob", True),
                   router_aux_loss_coef=tc.get("router_aux_loss_coef", 0.0)) if tc.get("model_type") == "qwen3_moe" else {}
        rope = tc.get("rope_parameters") or {}
        t = InternVLTextConfig(
            num_layers=tc.get("num_hidden_layers", 28), hidden_size=tc.get("hidden_size", 3584),
            intermediate_size=tc.get("intermediate_size", 18944), num_attention_heads=tc.get("num_attention_heads", 28),
            num_key_value_heads=tc.get("num_key_value_heads", 4), head_dim=tc.get("head_dim"),
            vocab_size=tc.get("vocab_size", 151674), rope_theta=tc.get("rope_theta", rope.get("rope_theta", 1e6)),
            rms_norm_eps=tc.get("rms_norm_eps", 1e-6), qk_norm=qwen3,
            qkv_bias=tc.get("attention_bias", not qwen3) if qwen3 else True,
            tie_word_embeddings=tc.get("tie_word_embeddings", hf.get("tie_word_embeddings", False)), **moe)
        return InternVLConfig(vision=v, text=t, downsample_ratio=hf.get("downsample_ratio", 0.5),
                              image_token_id=hf.get("image_token_id", 151667))


def _norm(kind: str, width: int, eps: float) -> nn.Module:
    return RMSNorm(width, eps) if kind == "rms_norm" else ops.LayerNorm(width, eps=eps)


class InternViTBlock(nn.Module):
    """x + lambda_1 * attn(norm(x)); x + lambda_2 * mlp(norm(x)).  Tiles are equal-length sequences, so attention runs
    on the dense [tiles, tokens, heads, head_dim] layout."""

    def __init__(self, c: InternViTConfig):
        super().__init__()
        self.num_heads, self.head_dim = c.num_heads, c.hidden_size // c.num_heads
        self.norm1 = _norm(c.norm_type, c.hidden_size, c.eps)
        self.norm2 = _norm(c.norm_type, c.hidden_size, c.eps)
        self.attn_qkv = Linear(c.hidden_size, 3 * c.hidden_size, bias=c.attention_bias)
        self.q_norm = RMSNorm(c.hidden_size, c.eps) if c.use_qk_norm else None
        self.k_norm = RMSNorm(c.hidden_size, c.eps) if c.use_qk_norm else None
        self.attn_proj = Linear(c.hidden_size, c.hidden_size)
        self.mlp_fc1 = Linear(c.hidden_size, c.intermediate_size)
        self.mlp_fc2 = Linear(c.intermediate_size, c.hidden_size)
        self.lambda_1 = nn.Parameter(torch.full((c.hidden_size,), c.layer_scale_init))
        self.lambda_2 = nn.Parameter(torch.full((c.hidden_size,), c.layer_scale_init))

    def forward(self, x):
        B, S, H = x.shape
        q, k, v = self.attn_qkv(self.norm1(x)).view(B, S, 3, H).unbind(2)
        if self.q_norm is not None:
            q, k = self.q_norm(q.contiguous()), self.k_norm(k.contiguous())
        shape = (B, S, self.num_heads, self.head_dim)
        o = ops.attention_dense(q.reshape(shape), k.reshape(shape), v.reshape(shape), causal=False)
        x = x + self.lambda_1.to(x.dtype) * self.attn_proj(o.reshape(B, S, H))
        return x + self.lambda_2.to(x.dtype) * self.mlp_fc2(ops.gelu(self.mlp_fc1(self.norm2(x))))


class InternViTEmbed(nn.Module):
    """Patch projection (a matmul over flattened patches), class token, absolute position table."""

    def __init__(self, c: InternViTConfig):
        super().__init__()
        self.c = c
        self.side = c.image_size // c.patch_size
        self.proj = Linear(c.in_channels * c.patch_size ** 2, c.hidden_size)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, c.hidden_size))
        self.position_embeddings = nn.Parameter(torch.zeros(1, self.side ** 2 + 1, c.hidden_size))

    def positions(self, gh: int, gw: int) -> torch.Tensor:
        pe = self.position_embeddings
        if gh == self.side and gw == self.side:
            return pe
        grid = pe[:, 1:].reshape(1, self.side, self.side, -1).permute(0, 3, 1, 2)
        grid = F.interpolate(grid.float(), size=(gh, gw), mode="bicubic", align_corners=False).to(pe.dtype)
        return torch.cat([pe[:, :1], grid.permute(0, 2, 3, 1).reshape(1, gh * gw, -1)], dim=1)

    def forward(self, pixel_values):
        c = self.c
        B, C, Hh, Ww = pixel_values.shape
        gh, gw, p = Hh // c.patch_size, Ww // c.patch_size, c.patch_size
        patches = pixel_values.view(B, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(B, gh * gw, C * p * p)
        x = self.proj(patches.to(self.proj.weight.dtype))
        x = torch.cat([self.cls_token.to(x.dtype).expand(B, -1, -1), x], dim=1)
        return x + self.positions(gh, gw).to(x.dtype)


def pixel_shuffle(x: torch.Tensor, ratio: float) -> torch.Tensor:
    """[B, W, H, C] -> [B, W * r, H * r, C / r^2] in the published checkpoint's element order."""
    B, W, Hh, C = x.shape
    x = x.reshape(B, W, int(Hh * ratio), int(C / ratio))
    x = x.permute(0, 2, 1, 3).reshape(B, int(Hh * ratio), int(W * ratio), int(C / (ratio * ratio)))
    return x.permute(0, 2, 1, 3)


class InternVLProjector(nn.Module):
    def __init__(self, vision_width: int, text_width: int, ratio: float):
        super().__init__()
        width = vision_width * int(1 / ratio) ** 2
        self.layer_norm = ops.LayerNorm(width, eps=1e-5)
        self.linear_1 = Linear(width, text_width)
        self.linear_2 = Linear(text_width, text_width)

    def forward(self, x):
        return self.linear_2(ops.gelu(self.linear_1(self.layer_norm(x))))


class InternViT(nn.Module):
    def __init__(self, c: InternViTConfig):
        super().__init__()
        self.c = c
        self.embed = InternViTEmbed(c)
        self.blocks = nn.ModuleList([InternViTBlock(c) for _ in range(c.depth)])

    def forward(self, pixel_values, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        x = run(self.embed, pixel_values)
        for b in self.blocks:
            x = run(b, x)
        return x


class InternVLConnector(nn.Module):
    """Tower output [tiles, 1 + gh * gw, C] -> text-width tokens [tiles * gh * gw * r^2, H_text]."""

    def __init__(self, cfg: InternVLConfig):
        super().__init__()
        v = cfg.vision
        self.ratio = cfg.downsample_ratio
        self.norm = ops.LayerNorm(v.hidden_size, eps=v.eps) if v.final_layernorm else None
        self.projector = InternVLProjector(v.hidden_size, cfg.text.hidden_size, cfg.downsample_ratio)

    def forward(self, x, gh: int, gw: int):
        if self.norm is not None:
            x = self.norm(x)
        B = x.shape[0]
        x = pixel_shuffle(x[:, 1:].reshape(B, gh, gw, -1), self.ratio)
        return self.projector(x.reshape(-1, x.shape[-1]))


def _seq_start(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """Start offset of the packed sequence every token belongs to."""
    cu = cu_seqlens.long()
    seq = torch.bucketize(torch.arange(total, device=cu.device), cu[1:], right=True)
    return cu[seq.clamp(max=cu.numel() - 2)]


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    f = positions.float().unsqueeze(-1) * inv
    emb = torch.cat((f, f), dim=-1)
    return emb.cos(), emb.sin()


@model_register.register("internvl")
@model_register.register("internvl3")
@model_register.register("internvl3_5")
class InternVLModel(nn.Module):
    """Packed-sequence InternVL3 / InternVL3.5 for training and generation.

    ``forward(batch)``: ``input_ids`` [T], shifted ``labels`` [T], ``cu_seqlens``, ``max_seqlen``, optional
    ``pixel_values`` [tiles, 3, H, W] (each tile fills ``tokens_per_tile`` image placeholders, in order) and optional 1-D
    ``position_ids`` [T] (default: positions restart at every packed sequence).  Returns ``(loss_sum, n_valid)`` or
    logits without labels."""

    config_class = InternVLConfig

    def __init__(self, config: Optional[InternVLConfig] = None, ep_size: Optional[int] = None):
        super().__init__()
        config = config or InternVLConfig.internvl3_5_8b()
        self.config = config
        t = config.text
        ep = ep_size if ep_size is not None else get_parallel_state().size("ep")
        if t.num_experts and t.num_experts % ep:
            raise ValueError(f"num_experts {t.num_experts} must be divisible by expert_parallel_size {ep}")
        self.visual = InternViT(config.vision)
        self.connector = InternVLConnector(config)
        self.embed_tokens = Embedding(t.vocab_size, t.hidden_size)
        sparse = t.num_experts > 0
        self.layers = nn.ModuleList([Qwen3DecoderLayer(t, sparse, t.num_experts // ep if sparse else None)
                                     for _ in range(t.num_layers)])
        self.lm_head = LMHead(t)
        blocks = [m for m in self.modules() if isinstance(m, SparseMoeBlock)]
        for b in blocks:                    # model-level auxiliary term = coef * mean over MoE layers
            b.aux_scale = t.router_aux_loss_coef / len(blocks)

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if "lambda_" in name:
                p.fill_(self.config.vision.layer_scale_init)
            elif p.dim() >= 2:
                p.copy_(_normal_like(p, self.config.init_std, g))
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)

    def fsdp_units(self) -> List[Tuple[str, nn.Module]]:
        units = [("embed_tokens", self.embed_tokens), ("visual.embed", self.visual.embed)]
        units += [(f"visual.blocks.{i}", b) for i, b in enumerate(self.visual.blocks)]
        units += [("connector", self.connector)]
        units += [(f"layers.{i}", l) for i, l in enumerate(self.layers)]
        units += [("lm_head", self.lm_head)]
        return units

    def expert_units(self):
        """Expert parameter units (sharded over the expert-FSDP group, gradients divided by the world size)."""
        return [(f"layers.{i}.mlp.experts", l.mlp.experts) for i, l in enumerate(self.layers) if l.sparse]

    def hf_ops(self):
        from ..checkpoint.hf import internvl_ops
        return internvl_ops(self.config)

    def aux_loss(self):
        """Value of the router load-balancing term of the last forward (its gradient is attached inside the blocks)."""
        ls = [l.mlp.aux_loss for l in self.layers if l.sparse and l.mlp.aux_loss is not None]
        return self.config.text.router_aux_loss_coef * torch.stack(ls).mean() if ls else None

    def image_features(self, pixel_values, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        p = self.config.vision.patch_size
        gh, gw = pixel_values.shape[-2] // p, pixel_values.shape[-1] // p
        return run(self.connector, self.visual(pixel_values, run=run), gh, gw)

    def forward(self, batch: dict, run=None, kv_cache: Optional[list] = None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        t = self.config.text
        ids = batch["input_ids"]
        x = run(self.embed_tokens, ids)
        pv = batch.get("pixel_values")
        if pv is not None and pv.numel() > 0:
            v = self.image_features(pv.to(x.dtype), run)
            img_pos = batch.get("image_positions")
            if img_pos is None:
                img_pos = (ids == self.config.image_token_id).nonzero(as_tuple=True)[0]
            if img_pos.numel() != v.shape[0]:
                raise ValueError(f"{img_pos.numel()} image placeholder tokens for {v.shape[0]} image features "
                                 f"({self.config.tokens_per_tile} per {self.config.vision.image_size}-pixel tile)")
            x = x.index_copy(0, img_pos, v.to(x.dtype))
        cos, sin = batch.get("rope_cos"), batch.get("rope_sin")
        if cos is None:
            pos = batch.get("position_ids")
            if pos is None or pos.dim() != 1:
                if kv_cache is not None:
                    past = kv_cache[0]["k"].shape[0] if "k" in kv_cache[0] else 0
                    pos = past + torch.arange(ids.shape[0], device=ids.device)
                else:
                    pos = torch.arange(ids.shape[0], device=ids.device) - _seq_start(batch["cu_seqlens"], ids.shape[0])
            cos, sin = rope_cos_sin(pos, t.head_dim, t.rope_theta)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        for i, layer in enumerate(self.layers):
            if kv_cache is not None:
                x = run(layer, x, cos, sin, None, 0, kv_cache[i])
            else:
                x = run(layer, x, cos, sin, batch["cu_seqlens"], batch["max_seqlen"])
        if kv_cache is not None and batch.get("labels") is None:
            x = x[-1:]
        return run(self.lm_head, x, batch.get("labels"))
