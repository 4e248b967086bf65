"""Unified understanding + generation models and the reward model.

* ``BagelMoT``      -- mixture-of-transformers decoder (mindspeed_mm/models/omni/mllms/bagel_qwen2_mot.py:157,318,468 and
  omni_model.py:13): every layer holds two parameter sets, one for "understanding" tokens (text, ViT features) and one for
  "generation" tokens (noised VAE latents); norms, q/k/v/o projections and MLPs are applied per set, attention is joint
  over the packed sample.  Losses: cross entropy on text positions, flow-matching MSE on latent positions.
* ``RewardModelBT`` -- a VLM backbone with a linear value head read at the last token of every sequence and the
  Bradley-Terry pairwise loss (mindspeed_mm/models/reward_model.py:17).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .composable import ComposableConfig, ComposableLM, DecoderConfig
from .qwen2_5_vl import Embedding, Linear, RMSNorm
from .registry import model_register
from .wan import sinusoidal_embedding

IGNORE = -100


@dataclass
class BagelConfig:
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_layers: int = 28
    num_heads: int = 28
    num_kv_heads: int = 4
    vocab_size: int = 152064
    rope_theta: float = 1e6
    eps: float = 1e-6
    latent_channels: int = 16
    latent_patch: int = 2
    max_latent_size: int = 64                 # side of the learned 2-D position table for latent patches
    vit_dim: int = 1152
    freq_dim: int = 256
    timestep_shift: float = 1.0
    ce_weight: float = 1.0
    mse_weight: float = 1.0
    freeze_und: bool = False

    @staticmethod
    def tiny(**kw):
        d = dict(hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4, num_kv_heads=2, vocab_size=128, latent_channels=4,
                 max_latent_size=8, vit_dim=24, freq_dim=16)
        d.update(kw)
        return BagelConfig(**d)


class _Set(nn.Module):
    """One parameter set of a layer (understanding or generation)."""

    def __init__(self, c: BagelConfig):
        super().__init__()
        H, hd = c.hidden_size, c.hidden_size // c.num_heads
        self.input_layernorm, self.post_attention_layernorm = RMSNorm(H, c.eps), RMSNorm(H, c.eps)
        self.qkv = Linear(H, (c.num_heads + 2 * c.num_kv_heads) * hd, bias=True)
        self.o_proj = Linear(c.num_heads * hd, H, bias=False)
        self.q_norm, self.k_norm = RMSNorm(hd, c.eps), RMSNorm(hd, c.eps)
        self.gate_up = Linear(H, 2 * c.intermediate_size, bias=False)
        self.down = Linear(c.intermediate_size, H, bias=False)


def _by_set(x, idx_und, idx_gen, f_und, f_gen, width=None):
    """Applies ``f_und`` / ``f_gen`` to the rows of ``x`` selected by the two index sets and scatters the results back."""
    yu = f_und(x[idx_und])
    out = x.new_zeros(x.shape[0], *(yu.shape[1:] if width is None else width))
    out = out.index_copy(0, idx_und, yu)
    if idx_gen.numel():
        out = out.index_copy(0, idx_gen, f_gen(x[idx_gen]))
    return out


class MoTLayer(nn.Module):
    def __init__(self, c: BagelConfig):
        super().__init__()
        self.c = c
        self.und, self.gen = _Set(c), _Set(c)

    def forward(self, x, idx_und, idx_gen, cos, sin, cu, max_len, masks=None):
        c = self.c
        nh, nkv, hd = c.num_heads, c.num_kv_heads, c.hidden_size // c.num_heads
        u, g = self.und, self.gen
        h = _by_set(x, idx_und, idx_gen, u.input_layernorm, g.input_layernorm)
        qkv = _by_set(h, idx_und, idx_gen, u.qkv, g.qkv)
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], -1)
        q, k, v = q.view(-1, nh, hd), k.view(-1, nkv, hd), v.view(-1, nkv, hd)
        q = _by_set(q, idx_und, idx_gen, u.q_norm, g.q_norm)
        k = _by_set(k, idx_und, idx_gen, u.k_norm, g.k_norm)
        if c.freeze_und:
            keep = torch.zeros(x.shape[0], 1, 1, dtype=torch.bool, device=x.device).index_fill(0, idx_gen, True)
            q, k, v = (torch.where(keep, t, t.detach()) for t in (q, k, v))
        q, k = ops.rope_rotate_half(q, cos, sin), ops.rope_rotate_half(k, cos, sin)
        if masks is None:
            o = ops.attention_varlen(q, k, v, cu, cu, max_len, max_len, causal=True)
        else:
            outs = []
            rep = nh // nkv
            for i, m in enumerate(masks):
                a, b = int(cu[i]), int(cu[i + 1])
                qi = q[a:b].transpose(0, 1)[None]
                ki = k[a:b].repeat_interleave(rep, 1).transpose(0, 1)[None]
                vi = v[a:b].repeat_interleave(rep, 1).transpose(0, 1)[None]
                outs.append(F.scaled_dot_product_attention(qi, ki, vi, attn_mask=m.to(q.device)[None, None])[0].transpose(0, 1))
            o = torch.cat(outs, 0)
        o = _by_set(o.reshape(-1, nh * hd), idx_und, idx_gen, u.o_proj, g.o_proj)
        x = x + o
        y = _by_set(x, idx_und, idx_gen,
                    lambda t: u.down(ops.swiglu(u.gate_up(u.post_attention_layernorm(t)))),
                    lambda t: g.down(ops.swiglu(g.gate_up(g.post_attention_layernorm(t)))))
        if c.freeze_und:
            keep = torch.zeros(x.shape[0], 1, dtype=torch.bool, device=x.device).index_fill(0, idx_gen, True)
            y = torch.where(keep, y, y.detach())
        return x + y


def bagel_attention_mask(modes: Sequence[str], lens: Sequence[int]) -> torch.Tensor:
    """Per-sample mask from consecutive splits: "causal" (text), "full" (ViT tokens: bidirectional inside the split),
    "noise" (latent tokens: bidirectional inside the split, and invisible to every later split, which conditions on
    the clean copy instead).  Every split sees all earlier visible splits."""
    L = sum(lens)
    m = torch.zeros(L, L, dtype=torch.bool)
    start = 0
    for mode, n in zip(modes, lens):
        end = start + n
        m[start:end, :start] = True
        if mode == "causal":
            m[start:end, start:end] = torch.tril(torch.ones(n, n, dtype=torch.bool))
        else:
            m[start:end, start:end] = True
        start = end
    start = 0
    for mode, n in zip(modes, lens):
        if mode == "noise":
            m[start + n:, start:start + n] = False
        start += n
    return m


@model_register.register("bagel")
class BagelMoT(nn.Module):
    """Packed batch keys: ``input_ids`` [T] (0 at non-text rows), ``text_rows`` [n_text], ``vit_rows`` + ``vit_embeds`` [n_vit,
    vit_dim], ``latent_rows`` + ``latents`` [n_lat, C * p * p] (clean) + ``latent_pos`` [n_lat] (index into the 2-D table) +
    ``timesteps`` [n_lat] in (0, 1) (sigma per token, after the shift), optional ``noise``; ``labels`` [T] for text rows,
    ``position_ids`` [T], ``cu_seqlens``, ``max_seqlen``, optional ``attention_masks`` (list of [L, L] bool).
    Returns ``dict(loss, ce, mse)``."""

    config_class = BagelConfig

    def __init__(self, config: Optional[BagelConfig] = None):
        super().__init__()
        self.config = c = config or BagelConfig.tiny()
        self.embed_tokens = Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(MoTLayer(c) for _ in range(c.num_layers))
        self.io = _BagelIO(c)

    def fsdp_units(self):
        return [("embed_tokens", self.embed_tokens), ("io", self.io)] + [(f"layers.{i}", l) for i, l in enumerate(self.layers)]

    def forward(self, batch: dict, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        dt = self.embed_tokens.weight.dtype
        T = batch["input_ids"].shape[0]
        dev = batch["input_ids"].device
        x = torch.zeros(T, c.hidden_size, dtype=dt, device=dev)
        text_rows = batch["text_rows"]
        x = x.index_copy(0, text_rows, run(self.embed_tokens, batch["input_ids"][text_rows]))
        und_rows = [text_rows]
        if batch.get("vit_rows") is not None and batch["vit_rows"].numel():
            x = x.index_copy(0, batch["vit_rows"], run(self.io, "vit", batch["vit_embeds"].to(dt)))
            und_rows.append(batch["vit_rows"])
        lat_rows = batch.get("latent_rows")
        target = None
        if lat_rows is not None and lat_rows.numel():
            clean = batch["latents"].to(dt)
            noise = batch.get("noise")
            if noise is None:
                noise = torch.randn_like(clean)
            sig = batch["timesteps"].to(dt)[:, None]
            noisy = (1 - sig) * clean + sig * noise
            target = (noise - clean).float()
            x = x.index_copy(0, lat_rows, run(self.io, "latent", noisy, batch["timesteps"], batch["latent_pos"]))
        else:
            lat_rows = torch.zeros(0, dtype=torch.long, device=dev)
        idx_und = torch.cat(und_rows).sort().values
        idx_gen = lat_rows
        hd = c.hidden_size // c.num_heads
        cos, sin = ops.ref.mrope_cos_sin(batch["position_ids"][None].expand(3, -1), hd, c.rope_theta, (hd // 2, 0, 0))
        cos, sin = cos.to(dt), sin.to(dt)
        for layer in self.layers:
            x = run(layer, x, idx_und, idx_gen, cos, sin, batch["cu_seqlens"], batch["max_seqlen"], batch.get("attention_masks"))
        out = dict(loss=None, ce=None, mse=None)
        total = x.new_zeros((), dtype=torch.float32)
        labels = batch.get("labels")
        if labels is not None:
            out["ce"] = run(self.io, "ce", x[text_rows], labels[text_rows])
            total = total + c.ce_weight * out["ce"]
        if target is not None:
            pred = run(self.io, "velocity", x[idx_gen]).float()
            out["mse"] = ((pred - target) ** 2).mean()
            out["pred_velocity"] = pred
            total = total + c.mse_weight * out["mse"]
        out["loss"] = total
        return total if batch.get("loss_only") else out


class _BagelIO(nn.Module):
    """Everything around the decoder stack, as one sharding unit with several entry points: ViT connector, latent
    input path (projection + timestep embedding + 2-D position table), text head with cross entropy, latent output head."""

    def __init__(self, c: BagelConfig):
        super().__init__()
        self.c = c
        H = c.hidden_size
        self.norm, self.norm_gen = RMSNorm(H, c.eps), RMSNorm(H, c.eps)
        self.lm_head = nn.Parameter(torch.empty(c.vocab_size, H))
        pd = c.latent_channels * c.latent_patch ** 2
        self.vae2llm, self.llm2vae = Linear(pd, H), Linear(H, pd)
        self.time_1, self.time_2 = Linear(c.freq_dim, H), Linear(H, H)
        self.latent_pos_embed = nn.Parameter(torch.zeros(c.max_latent_size ** 2, H))
        self.connector_1, self.connector_2 = Linear(c.vit_dim, H), Linear(H, H)

    def forward(self, mode: str, *a):
        if mode == "vit":
            return self.connector_2(ops.gelu_tanh(self.connector_1(a[0])))
        if mode == "latent":
            noisy, timesteps, pos = a
            dt = noisy.dtype
            temb = self.time_2(F.silu(self.time_1(sinusoidal_embedding(timesteps.float() * 1000.0, self.c.freq_dim).to(dt))))
            return self.vae2llm(noisy) + temb + self.latent_pos_embed[pos].to(dt)
        if mode == "ce":
            s, n = ops.linear_cross_entropy(self.norm(a[0]), self.lm_head, a[1])
            return s / n.clamp(min=1).to(s.dtype)
        if mode == "velocity":
            return self.llm2vae(self.norm_gen(a[0]))
        raise ValueError(mode)


# ------------------------------------------------------------------------------------------------- reward model
class _ValueHead(nn.Module):
    """Final norm of the decoder (its vocabulary table is dropped) followed by the linear value head."""

    def __init__(self, lm_head: nn.Module, hidden: int, output_dim: int):
        super().__init__()
        self.lm_head = lm_head
        self.lm_head.weight = None
        self.rm_head = nn.Linear(hidden, output_dim, bias=False)

    def forward(self, h):
        return self.rm_head(self.lm_head.norm(h).to(self.rm_head.weight.dtype))


@model_register.register("qwen2vl_reward")
class RewardModelBT(nn.Module):
    """``forward(batch)``: packed VLM batch whose sequences alternate chosen, rejected; the value head is read at the last
    token of every sequence (or at the last occurrence of ``reward_token_id`` when one is configured)."""

    def __init__(self, backbone: Optional[ComposableLM] = None, output_dim: int = 1, reward_token_id: Optional[int] = None):
        super().__init__()
        if backbone is None:
            from .composable import build_preset
            backbone = build_preset("qwen2vl")
        self.backbone = backbone
        self.reward_token_id = reward_token_id
        self.value_head = _ValueHead(backbone.lm_head, backbone.config.text.hidden_size, output_dim)

    def fsdp_units(self):
        return [(f"backbone.{n}", m) for n, m in self.backbone.fsdp_units() if n != "lm_head"] + [("value_head", self.value_head)]

    def rewards(self, batch: dict, run=None) -> torch.Tensor:
        run = run or (lambda m, *a, **k: m(*a, **k))
        b = {k: v for k, v in batch.items() if k != "labels"}
        b["return_hidden"] = True
        h = self.backbone(b, run)
        cu = batch["cu_seqlens"].long()
        rows = cu[1:] - 1
        if self.reward_token_id is not None:
            ids = batch["input_ids"]
            hit = (ids == self.reward_token_id).nonzero(as_tuple=True)[0]
            seq_of = torch.bucketize(hit, cu[1:], right=True)
            for s in range(rows.numel()):
                mine = hit[seq_of == s]
                if mine.numel():
                    rows[s] = mine[-1]
        return run(self.value_head, h[rows]).squeeze(-1)

    def forward(self, batch: dict, run=None):
        from ..tasks.preference import bradley_terry_loss
        r = self.rewards(batch, run)
        chosen, rejected = r[0::2], r[1::2]
        self.last_accuracy = (chosen > rejected).float().mean().detach()
        return bradley_terry_loss(chosen.float(), rejected.float())
