"""Variants of the Wan DiT that reuse its blocks: Wan2.2 (TI2V per-token timesteps, token-routed MoE FFN, the
high-noise / low-noise expert pair) and VACE (control branch whose hints are added to chosen trunk layers).

Reference: mindspeed_mm/fsdp/models/wan2_2/modeling_wan2_2.py (``WanMoERouter`` :483, ``WanSparseMoEBlock`` :570,
``WanModel.forward`` :813 with per-token ``t``), wan2_2/diffusion.py:21 (timestep boundaries that assign a noise range to
each expert), mindspeed_mm/models/predictor/dits/vace.py (``VaceWanAttentionBlock`` :17, ``VaceDit`` :51, ``VACEModel`` :202).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .qwen2_5_vl import Linear
from .registry import model_register
from .wan import WanBlock, WanConfig, WanDiT, WanEmbeddings, WanHead, sinusoidal_embedding


@dataclass
class Wan22Config(WanConfig):
    moe_num_experts: int = 0          # > 0: the dense FFN of every block becomes top-k routed experts
    moe_top_k: int = 1
    per_token_timestep: bool = False  # TI2V: every latent token carries its own timestep (clean first frame = 0)

    @staticmethod
    def ti2v_5b():
        return Wan22Config(model_type="ti2v", in_dim=48, out_dim=48, hidden_size=3072, ffn_dim=14336, num_heads=24, num_layers=30,
                           per_token_timestep=True)

    @staticmethod
    def a14b(model_type: str = "t2v"):
        return Wan22Config(model_type=model_type, in_dim=16 if model_type == "t2v" else 36)

    @staticmethod
    def tiny(**kw):
        d = dict(hidden_size=128, ffn_dim=256, num_heads=4, num_layers=2, text_dim=64, text_len=16, freq_dim=32)
        d.update(kw)
        return Wan22Config(**d)

    @staticmethod
    def from_mm_json(pred: dict) -> "Wan22Config":
        keys = Wan22Config.__dataclass_fields__.keys()
        return Wan22Config(**{k: v for k, v in pred.items() if k in keys})


class WanMoEFFN(nn.Module):
    """Softmax router over ``E`` experts, top-k, SwiGLU experts stored as two stacked tensors so the
    grouped GEMM (and expert parallelism, which shards dim 0) applies."""

    def __init__(self, c: Wan22Config):
        super().__init__()
        self.top_k, self.E = c.moe_top_k, c.moe_num_experts
        self.router = nn.Linear(c.hidden_size, self.E, bias=False)
        self.gate_up = nn.Parameter(torch.empty(self.E, c.hidden_size, 2 * c.ffn_dim))
        self.down = nn.Parameter(torch.empty(self.E, c.ffn_dim, c.hidden_size))
        nn.init.normal_(self.gate_up, std=c.init_std)
        nn.init.normal_(self.down, std=c.init_std)

    def forward(self, x):
        B, S, H = x.shape
        flat = x.reshape(B * S, H)
        probs = F.softmax(self.router(flat).float(), -1)
        w, ids = probs.topk(self.top_k, -1)
        w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
        return ops.moe_experts(flat, ids, w, self.gate_up, self.down).reshape(B, S, H)


class Wan22Block(WanBlock):
    def __init__(self, c: Wan22Config):
        super().__init__(c)
        self.moe = None
        if c.moe_num_experts > 0:
            del self.ffn_0, self.ffn_2
            self.moe = WanMoEFFN(c)

    def _ffn(self, h):
        return self.moe(h) if self.moe is not None else self.ffn_2(ops.gelu_tanh(self.ffn_0(h)))

    def forward(self, x, time_emb, ctx, rope_cos, rope_sin, seq_sizes=None, n_img: int = 0, rope_full=None):
        if time_emb.dim() == 3 and self.moe is None:
            return super().forward(x, time_emb, ctx, rope_cos, rope_sin, seq_sizes, n_img, rope_full)
        if time_emb.dim() == 3:
            time_emb = time_emb[:, None]                                          # [B, 1, 6, H]
        e = (self.modulation.to(time_emb.dtype)[:, None] + time_emb).unbind(2)    # 6 x [B, S or 1, H]
        mod = lambda h, sc, sh: ops.layer_norm(h, None, None, self.eps) * (1 + sc) + sh       # noqa: E731
        y = self.self_attn(mod(x, e[1], e[0]), (rope_cos, rope_sin), seq_sizes, rope_full)
        x = x + y * e[2]
        x = x + self.cross_attn(self.norm3(x), ctx, n_img)
        y = self._ffn(mod(x, e[4], e[3]))
        return x + y * e[5]


class Wan22Embeddings(WanEmbeddings):
    def forward(self, latents, timestep, prompt, clip_feature=None):
        if timestep.dim() == 1:
            return super().forward(latents, timestep, prompt, clip_feature)
        # per-token timesteps [B, S]: embed every distinct value once (a TI2V batch has two: 0 and t)
        dtype = self.patch_embedding.weight.dtype
        B, S = timestep.shape
        uniq, inv = torch.unique(timestep.reshape(-1), return_inverse=True)
        te = sinusoidal_embedding(uniq, self.c.freq_dim).to(dtype)
        times_u = self.time_embedding_2(F.silu(self.time_embedding_0(te)))
        proj_u = self.time_projection(F.silu(times_u))
        times = times_u[inv].view(B, S, -1)
        time_emb = proj_u[inv].view(B, S, 6, -1)
        x, _, _, ctx, n_img = super().forward(latents, timestep[:, -1], prompt, clip_feature)
        return x, times, time_emb, ctx, n_img


class Wan22Head(WanHead):
    def forward(self, x, times):
        if times.dim() == 2:
            return super().forward(x, times)
        e = (self.modulation.to(times.dtype)[:, None] + times[:, :, None]).unbind(2)          # 2 x [B, S, H]
        return self.head(ops.layer_norm(x, None, None, self.c.eps) * (1 + e[1]) + e[0])


@model_register.register("wan2_2")
class Wan22DiT(WanDiT):
    """Wan2.2 trunk.  ``timestep`` is ``[B]`` or, for TI2V, ``[B, tokens]``; ``ti2v_timesteps`` builds the latter."""
    config_class = Wan22Config

    def __init__(self, config: Wan22Config):
        nn.Module.__init__(self)
        self.config = config
        self.embeddings = Wan22Embeddings(config)
        self.blocks = nn.ModuleList([Wan22Block(config) for _ in range(config.num_layers)])
        self.head = Wan22Head(config)

    def ti2v_timesteps(self, latents, timestep, first_frame_clean: bool = True):
        pf, ph, pw = self.config.patch_size
        f, h, w = latents.shape[2] // pf, latents.shape[3] // ph, latents.shape[4] // pw
        t = timestep.reshape(-1, 1, 1).expand(latents.shape[0], f, h * w).clone().float()
        if first_frame_clean:
            t[:, 0] = 0
        return t.reshape(latents.shape[0], f * h * w)

    def forward(self, latents, timestep, prompt, clip_feature=None, run=None, first_frame_clean: bool = False):
        if self.config.per_token_timestep and timestep.dim() == 1 and first_frame_clean:
            timestep = self.ti2v_timesteps(latents, timestep)
        return super().forward(latents, timestep, prompt, clip_feature, run)


@model_register.register("wan2_2_a14b")
class WanExpertPair(nn.Module):
    """The two-expert denoiser of Wan2.2-A14B: one full DiT for the noisy end of the trajectory, one for the clean end.
    ``boundary`` is the switch point as a fraction of the training timesteps (0.875 text-to-video, 0.9 image-to-video).
    Training touches one expert per step (the scheduler's timestep boundaries pick the range); sampling routes each call
    by its timestep, so the pair behaves as a single ``model(latents, t, prompt)``."""
    config_class = Wan22Config

    def __init__(self, config: Wan22Config, boundary: Optional[float] = None, num_train_timesteps: int = 1000):
        super().__init__()
        self.config = config
        self.boundary = boundary if boundary is not None else (0.875 if config.model_type == "t2v" else 0.9)
        self.T = num_train_timesteps
        self.high_noise, self.low_noise = Wan22DiT(config), Wan22DiT(config)

    def expert_for(self, timestep) -> "Wan22DiT":
        t = float(timestep.reshape(-1)[0]) if torch.is_tensor(timestep) else float(timestep)
        return self.high_noise if t >= self.boundary * self.T else self.low_noise

    def scheduler_boundaries(self, which: str, shift: float = 5.0) -> Tuple[float, float]:
        """``(min_timestep_boundary, max_timestep_boundary)`` for the flow-match scheduler, whose training grid is indexed
        from the noisiest step and warped by ``sigma = shift * s / (1 + (shift - 1) * s)``: the high-noise expert owns the
        indices whose sigma is >= ``boundary`` (0.417 of the grid at boundary 0.875, 0.357 at 0.9, shift 5)."""
        b = self.boundary
        frac = 1.0 - b / (shift - (shift - 1.0) * b)
        return (0.0, frac) if which == "high" else (frac, 1.0)

    def fsdp_units(self):
        return [(f"high_noise.{n}", m) for n, m in self.high_noise.fsdp_units()] + \
               [(f"low_noise.{n}", m) for n, m in self.low_noise.fsdp_units()]

    def forward(self, latents, timestep, prompt, clip_feature=None, run=None):
        return self.expert_for(timestep)(latents, timestep, prompt, clip_feature, run)


# ------------------------------------------------------------------------------------------------- VACE
@dataclass
class VaceConfig(WanConfig):
    vace_layers: Sequence[int] = (0, 2, 4, 6, 8, 10, 12, 14, 16, 18, 20, 22, 24, 26, 28)
    vace_in_dim: int = 96

    @staticmethod
    def tiny(**kw):
        d = dict(hidden_size=128, ffn_dim=256, num_heads=4, num_layers=4, text_dim=64, text_len=16, freq_dim=32,
                 vace_layers=(0, 2), vace_in_dim=20)
        d.update(kw)
        return VaceConfig(**d)

    @staticmethod
    def from_mm_json(pred: dict) -> "VaceConfig":
        keys = VaceConfig.__dataclass_fields__.keys()
        return VaceConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in pred.items() if k in keys})


class VaceBlock(nn.Module):
    """A Wan block of the control branch.  The first one mixes the control tokens with the trunk's tokens; every
    one emits a projected copy of its state as the hint for its trunk layer."""

    def __init__(self, c: VaceConfig, first: bool):
        super().__init__()
        self.block = WanBlock(c)
        self.before_proj = Linear(c.hidden_size, c.hidden_size) if first else None
        self.after_proj = Linear(c.hidden_size, c.hidden_size)
        for lin in (self.before_proj, self.after_proj):
            if lin is not None:
                nn.init.zeros_(lin.weight)
                nn.init.zeros_(lin.bias)

    def forward(self, ctrl, x, time_emb, ctx, cos, sin):
        if self.before_proj is not None:
            ctrl = self.before_proj(ctrl) + x
        ctrl = self.block(ctrl, time_emb, ctx, cos, sin)
        return ctrl, self.after_proj(ctrl)


@model_register.register("vace")
class VaceWanDiT(WanDiT):
    """``forward(latents, timestep, prompt, vace_context=[B, vace_in_dim, F, H, W], vace_scale=1.0)``.  The trunk may be
    frozen (``freeze_trunk``) so that only the control branch trains, as the reference's VACE recipe does."""
    config_class = VaceConfig

    def __init__(self, config: VaceConfig):
        super().__init__(config)
        p = config.patch_size
        self.vace_patch_embedding = Linear(config.vace_in_dim * p[0] * p[1] * p[2], config.hidden_size)
        self.vace_blocks = nn.ModuleList([VaceBlock(config, i == 0) for i in range(len(config.vace_layers))])
        self.vace_to_trunk = {layer: i for i, layer in enumerate(config.vace_layers)}

    def fsdp_units(self):
        return super().fsdp_units() + [("vace_patch_embedding", self.vace_patch_embedding)] + \
               [(f"vace_blocks.{i}", b) for i, b in enumerate(self.vace_blocks)]

    def freeze_trunk(self):
        for name, p in self.named_parameters():
            p.requires_grad_(name.startswith("vace_"))

    def forward(self, latents, timestep, prompt, clip_feature=None, run=None, vace_context=None, vace_scale: float = 1.0):
        run = run or (lambda m, *a, **k: m(*a, **k))
        c = self.config
        x, times, time_emb, ctx, n_img = run(self.embeddings, latents, timestep, prompt, clip_feature)
        pf, ph, pw = c.patch_size
        grid = (latents.shape[2] // pf, latents.shape[3] // ph, latents.shape[4] // pw)
        cos, sin = ops.ref.rope3d_freqs(grid, c.hidden_size // c.num_heads, c.rope_theta, device=x.device)
        if x.shape[0] > 1:
            cos, sin = cos.repeat(x.shape[0], 1), sin.repeat(x.shape[0], 1)
        hints = []
        if vace_context is not None:
            tok, _ = self.embeddings.patchify(vace_context.to(x.dtype))
            ctrl = run(self.vace_patch_embedding, tok)
            if ctrl.shape[1] < x.shape[1]:                                       # shorter control clips are zero-padded
                ctrl = F.pad(ctrl, (0, 0, 0, x.shape[1] - ctrl.shape[1]))
            for vb in self.vace_blocks:
                ctrl, hint = run(vb, ctrl, x, time_emb, ctx, cos, sin)
                hints.append(hint)
        for i, blk in enumerate(self.blocks):
            x = run(blk, x, time_emb, ctx, cos, sin, None, n_img)
            if hints and i in self.vace_to_trunk:
                x = x + hints[self.vace_to_trunk[i]] * vace_scale
        return self.head.unpatchify(run(self.head, x, times), grid)
