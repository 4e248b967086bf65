"""Qwen3-VL (dense and MoE): vision tower with interpolated position embeddings and DeepStack, interleaved mRoPE text
decoder with per-head q/k RMSNorm, dense SwiGLU or top-k routed experts.

Reference: mindspeed_mm/fsdp/models/qwen3vl/modeling_qwen3_vl_moe.py (router :110-117, fused experts :125-126,
DeepStack :719-726,886-894) and the upstream Hugging Face modeling it derives from.  Differences from Qwen2.5-VL that
matter for weights and numerics:

* vision: patch 16, LayerNorm (affine) instead of RMSNorm, GELU(tanh) fc1/fc2 MLP, no window attention (one sequence per
  image frame), a learned 48 x 48 position table bilinearly interpolated to each image's patch grid, and DeepStack:
  the hidden states after vision layers ``deepstack_visual_indexes`` go through their own mergers and are ADDED to the
  hidden states of the first decoder layers at the visual token positions
* text: q/k RMSNorm per head before RoPE, no QKV bias, mRoPE with the (t, h, w) frequency bands interleaved
  (t h w t h w ... t t) instead of chunked
* MoE: ``softmax(fp32) -> top-k -> renormalise``; experts fused as ``gate_up_proj [E, H, 2F]`` / ``down_proj [E, F, H]``
  (the checkpoint layout; ``x @ W`` form)

Packed-sequence training interface of ``Qwen25VLModel``: ``forward(batch, run)`` -> ``(loss_sum, n_valid)`` or logits.
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
from .qwen2_5_vl import Embedding, Linear, LMHead, RMSNorm, _normal_like, vision_rot_pos_ids
from .registry import model_register


@dataclass
class Qwen3VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 2048
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: Sequence[int] = (8, 16, 24)
    eps: float = 1e-6
    window_size: int = 0             # no window attention; kept so that collators written for Qwen2.5-VL can read it


@dataclass
class Qwen3TextConfig(MoETextConfig):
    qkv_bias: bool = False
    mrope_interleaved: bool = True
    mrope_section: Sequence[int] = (24, 20, 20)
    rope_theta: float = 5000000.0
    num_experts: int = 0             # 0: dense SwiGLU FFN of ``intermediate_size``
    decoder_sparse_step: int = 1
    mlp_only_layers: Sequence[int] = ()


@dataclass
class Qwen3VLConfig:
    vision: Qwen3VisionConfig = field(default_factory=Qwen3VisionConfig)
    text: Qwen3TextConfig = field(default_factory=Qwen3TextConfig)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    vision_end_token_id: int = 151653
    init_std: float = 0.02

    def vision_plan(self, grid_thw: torch.Tensor) -> dict:
        """Host-side index plan of the vision tower (read by the packing collator)."""
        return qwen3_vision_plan(self.vision, grid_thw)

    def rope_index(self, input_ids: torch.Tensor, image_grid_thw=None, video_grid_thw=None):
        """mRoPE position ids [3, S] of one sample and the offset of the text that follows it."""
        return qwen3_rope_index(input_ids, image_grid_thw, video_grid_thw, self.image_token_id, self.video_token_id,
                                self.vision.spatial_merge_size)

    def layer_is_sparse(self, i: int) -> bool:
        t = self.text
        return bool(t.num_experts) and i not in t.mlp_only_layers and (i + 1) % t.decoder_sparse_step == 0

    @staticmethod
    def qwen3_vl_30b_a3b():
        return Qwen3VLConfig(
            vision=Qwen3VisionConfig(),
            text=Qwen3TextConfig(num_layers=48, hidden_size=2048, intermediate_size=6144, num_attention_heads=32,
                                 num_key_value_heads=4, head_dim=128, vocab_size=151936, num_experts=128,
                                 num_experts_per_tok=8, moe_intermediate_size=768))

    @staticmethod
    def qwen3_vl_8b():
        return Qwen3VLConfig(
            vision=Qwen3VisionConfig(out_hidden_size=4096),
            text=Qwen3TextConfig(num_layers=36, hidden_size=4096, intermediate_size=12288, num_attention_heads=32,
                                 num_key_value_heads=8, head_dim=128, vocab_size=151936))

    @staticmethod
    def tiny(moe: bool = True):
        return Qwen3VLConfig(
            vision=Qwen3VisionConfig(depth=3, hidden_size=128, intermediate_size=256, num_heads=4, out_hidden_size=256,
                                     num_position_embeddings=64, deepstack_visual_indexes=(0, 1)),
            text=Qwen3TextConfig(num_layers=3, hidden_size=256, intermediate_size=512, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, vocab_size=32000, mrope_section=(12, 10, 10),
                                 num_experts=8 if moe else 0, num_experts_per_tok=2, moe_intermediate_size=128),
            image_token_id=31999, video_token_id=31998, vision_start_token_id=31997, vision_end_token_id=31996)

    @staticmethod
    def from_hf(hf: dict) -> "Qwen3VLConfig":
        """From a Hugging Face ``config.json`` (``qwen3_vl`` / ``qwen3_vl_moe``)."""
        v, t = hf.get("vision_config", {}), hf.get("text_config", hf)
        rp = t.get("rope_parameters") or t.get("rope_scaling") or {}
        vis = Qwen3VisionConfig(
            depth=v.get("depth", 27), hidden_size=v.get("hidden_size", 1152), intermediate_size=v.get("intermediate_size", 4304),
            num_heads=v.get("num_heads", 16), in_channels=v.get("in_channels", 3), patch_size=v.get("patch_size", 16),
            temporal_patch_size=v.get("temporal_patch_size", 2), spatial_merge_size=v.get("spatial_merge_size", 2),
            out_hidden_size=v.get("out_hidden_size", t.get("hidden_size", 2048)),
            num_position_embeddings=v.get("num_position_embeddings", 2304),
            deepstack_visual_indexes=tuple(v.get("deepstack_visual_indexes", (8, 16, 24))))
        txt = Qwen3TextConfig(
            num_layers=t["num_hidden_layers"], hidden_size=t["hidden_size"], intermediate_size=t.get("intermediate_size", 0),
            num_attention_heads=t["num_attention_heads"], num_key_value_heads=t["num_key_value_heads"],
            head_dim=t.get("head_dim") or t["hidden_size"] // t["num_attention_heads"], vocab_size=t["vocab_size"],
            rms_norm_eps=t.get("rms_norm_eps", 1e-6), rope_theta=rp.get("rope_theta", t.get("rope_theta", 5e6)),
            mrope_section=tuple(rp.get("mrope_section", (24, 20, 20))), qkv_bias=t.get("attention_bias", False),
            num_experts=t.get("num_experts", t.get("num_local_experts", 0)), num_experts_per_tok=t.get("num_experts_per_tok", 8),
            moe_intermediate_size=t.get("moe_intermediate_size", 768), norm_topk_prob=t.get("norm_topk_prob", True),
            router_aux_loss_coef=t.get("router_aux_loss_coef", 0.0),
            decoder_sparse_step=t.get("decoder_sparse_step", 1), mlp_only_layers=tuple(t.get("mlp_only_layers", ())),
            tie_word_embeddings=hf.get("tie_word_embeddings", t.get("tie_word_embeddings", False)))
        return Qwen3VLConfig(vision=vis, text=txt, image_token_id=hf.get("image_token_id", 151655),
                             video_token_id=hf.get("video_token_id", 151656),
                             vision_start_token_id=hf.get("vision_start_token_id", 151652),
                             vision_end_token_id=hf.get("vision_end_token_id", 151653))


# ------------------------------------------------------------------------------------------ rotary tables
def interleaved_mrope_cos_sin(position_ids: torch.Tensor, head_dim: int, theta: float, section: Sequence[int]):
    """cos / sin [T, head_dim] for mRoPE with interleaved frequency bands: band i takes the temporal position, except
    bands 1, 4, 7 ... (< 3 * section[1]) which take the height and bands 2, 5, 8 ... (< 3 * section[2]) the width."""
    pos = position_ids.float()                                             # [3, T]
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=pos.device) / head_dim))
    freqs = pos.unsqueeze(-1) * inv                                        # [3, T, D/2]
    out = freqs[0].clone()
    for dim, off in ((1, 1), (2, 2)):
        idx = slice(off, section[dim] * 3, 3)
        out[..., idx] = freqs[dim][..., idx]
    emb = torch.cat((out, out), dim=-1)
    return emb.cos(), emb.sin()


def qwen3_rope_index(input_ids: torch.Tensor, image_grid_thw, video_grid_thw, image_token_id: int, video_token_id: int,
                     merge: int = 2) -> Tuple[torch.Tensor, int]:
    """mRoPE (t, h, w) position ids for ONE sample ([S] ids) -> ([3, S], delta).

    Text advances all three axes together.  Every run of image tokens takes the next image grid; a video is a run per
    FRAME (frames are separated by timestamp text), so its grid is split into ``t`` grids of one frame.  A visual block
    starting at position ``p`` has temporal position ``p`` for all its tokens, rows ``p .. p + h/merge - 1`` and
    columns ``p .. p + w/merge - 1``; the text after it restarts at ``p + max(h, w) / merge``."""
    ids = input_ids.tolist()
    S = len(ids)
    grids = {image_token_id: iter(image_grid_thw.tolist() if image_grid_thw is not None else ()),
             video_token_id: iter([[1, h, w] for t, h, w in (video_grid_thw.tolist() if video_grid_thw is not None else ())
                                   for _ in range(t)])}
    pos = torch.zeros(3, S, dtype=torch.long)
    cur, i = 0, 0
    while i < S:
        tok = ids[i]
        if tok in grids:
            t, h, w = next(grids[tok])
            gh, gw = h // merge, w // merge
            n = t * gh * gw
            if ids[i:i + n] != [tok] * n:
                raise ValueError(f"visual token run at {i} is shorter than its grid ({t}, {h}, {w}) needs ({n} tokens)")
            pos[0, i:i + n] = cur
            pos[1, i:i + n] = cur + torch.arange(gh).repeat_interleave(gw).repeat(t)
            pos[2, i:i + n] = cur + torch.arange(gw).repeat(t * gh)
            cur += max(gh, gw)
            i += n
        else:
            j = i
            while j < S and ids[j] not in grids:
                j += 1
            pos[:, i:j] = cur + torch.arange(j - i)
            cur += j - i
            i = j
    return pos, cur - S


# ------------------------------------------------------------------------------------------ vision tower
class Qwen3VisionBlock(nn.Module):
    def __init__(self, c: Qwen3VisionConfig):
        super().__init__()
        self.num_heads, self.head_dim = c.num_heads, c.hidden_size // c.num_heads
        self.norm1 = ops.LayerNorm(c.hidden_size, eps=c.eps)
        self.norm2 = ops.LayerNorm(c.hidden_size, eps=c.eps)
        self.attn_qkv = Linear(c.hidden_size, 3 * c.hidden_size)
        self.attn_proj = Linear(c.hidden_size, c.hidden_size)
        self.mlp_fc1 = Linear(c.hidden_size, c.intermediate_size)
        self.mlp_fc2 = Linear(c.intermediate_size, c.hidden_size)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        T = x.shape[0]
        q, k, v = self.attn_qkv(self.norm1(x)).view(T, 3, self.num_heads, self.head_dim).unbind(1)
        q = ops.rope_rotate_half(q, cos, sin)
        k = ops.rope_rotate_half(k, cos, sin)
        o = ops.attention_varlen(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=False)
        x = x + self.attn_proj(o.reshape(T, -1))
        return x + self.mlp_fc2(ops.gelu_tanh(self.mlp_fc1(self.norm2(x))), value_unused_in_backward=True)


class Qwen3PatchMerger(nn.Module):
    """LayerNorm (before or after the 2 x 2 regroup) -> fc1 -> GELU -> fc2.  The main merger normalises each patch
    (width ``hidden``); the DeepStack mergers normalise the regrouped row (width ``4 * hidden``)."""

    def __init__(self, c: Qwen3VisionConfig, postshuffle_norm: bool = False):
        super().__init__()
        self.width = c.hidden_size * c.spatial_merge_size ** 2
        self.postshuffle = postshuffle_norm
        self.norm = ops.LayerNorm(self.width if postshuffle_norm else c.hidden_size, eps=c.eps)
        self.fc1 = Linear(self.width, self.width)
        self.fc2 = Linear(self.width, c.out_hidden_size)

    def forward(self, x):
        x = self.norm(x.view(-1, self.width)) if self.postshuffle else self.norm(x).view(-1, self.width)
        return self.fc2(ops.gelu(self.fc1(x)))


class Qwen3PatchEmbed(nn.Module):
    """Conv3d(kernel = stride = (tp, p, p), bias) on pre-flattened patches (one GEMM) plus the interpolated learned
    position table, which the collator or ``plan`` hands over as gather indices and bilinear weights."""

    def __init__(self, c: Qwen3VisionConfig):
        super().__init__()
        self.in_dim = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        self.merge = c.spatial_merge_size
        self.proj = Linear(self.in_dim, c.hidden_size, bias=True)
        self.pos_embed = Embedding(c.num_position_embeddings, c.hidden_size)

    def forward(self, pixel_values, pos_idx, pos_wt):
        if pixel_values.shape[-1] != self.in_dim:
            raise ValueError(f"pixel_values rows are {pixel_values.shape[-1]} wide; this tower takes {self.in_dim} "
                             f"(channels x temporal patch x patch x patch)")
        x = self.proj(pixel_values)
        # four corner rows of the table per patch, weighted: [T, 4, H] * [T, 4, 1] -> [T, H]
        pe = (F.embedding(pos_idx, self.pos_embed.weight) * pos_wt.to(x.dtype).unsqueeze(-1)).sum(1)
        return x + pe


def position_table_plan(side: int, grid_thw: torch.Tensor, merge: int):
    """Gather indices [T, 4] and bilinear weights [T, 4] that turn the learned ``side x side`` table into per-patch
    position embeddings for every image, in the merge order of the patch sequence (host arithmetic)."""
    idxs, wts = [], []
    for t, h, w in grid_thw.tolist():
        hi, wi = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
        hf, wf = hi.int(), wi.int()
        hc, wc = (hf + 1).clamp(max=side - 1), (wf + 1).clamp(max=side - 1)
        dh, dw = hi - hf, wi - wf
        idx = torch.stack([hf[:, None] * side + wf[None], hf[:, None] * side + wc[None],
                           hc[:, None] * side + wf[None], hc[:, None] * side + wc[None]], -1)          # [h, w, 4]
        wt = torch.stack([(1 - dh)[:, None] * (1 - dw)[None], (1 - dh)[:, None] * dw[None],
                          dh[:, None] * (1 - dw)[None], dh[:, None] * dw[None]], -1)
        for a, store in ((idx.long(), idxs), (wt, wts)):
            a = a.view(h // merge, merge, w // merge, merge, 4).permute(0, 2, 1, 3, 4).reshape(-1, 4)
            store.append(a.repeat(t, 1))
    return torch.cat(idxs), torch.cat(wts)


def qwen3_vision_plan(c: Qwen3VisionConfig, grid_thw: torch.Tensor) -> dict:
    """Host arithmetic for a batch of images: 2-D rotary tables in merge order, one attention sequence per frame,
    and the gather plan of the interpolated position table."""
    head_dim = c.hidden_size // c.num_heads
    pos = vision_rot_pos_ids(grid_thw, c.spatial_merge_size)
    inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim // 2, 2, dtype=torch.float32) / (head_dim // 2)))
    freqs = (pos.unsqueeze(-1).float() * inv).flatten(1)
    emb = torch.cat((freqs, freqs), -1)
    lens = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])
    side = int(round(c.num_position_embeddings ** 0.5))
    pidx, pwt = position_table_plan(side, grid_thw, c.spatial_merge_size)
    return dict(cos=emb.cos(), sin=emb.sin(), cu_full=F.pad(lens.cumsum(0), (1, 0)).to(torch.int32),
                max_full=int(lens.max()), pos_idx=pidx, pos_wt=pwt, n_tokens=int(pos.shape[0]))


class Qwen3VisionTransformer(nn.Module):
    def __init__(self, c: Qwen3VisionConfig):
        super().__init__()
        self.cfg = c
        self.patch_embed = Qwen3PatchEmbed(c)
        self.blocks = nn.ModuleList([Qwen3VisionBlock(c) for _ in range(c.depth)])
        self.merger = Qwen3PatchMerger(c)
        self.deepstack_mergers = nn.ModuleList([Qwen3PatchMerger(c, True) for _ in c.deepstack_visual_indexes])

    @torch.no_grad()
    def plan(self, grid_thw: torch.Tensor, device) -> dict:
        """Index tensors for a batch of images, on ``device`` (the collator precomputes the same on the host)."""
        return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in qwen3_vision_plan(self.cfg, grid_thw).items()}

    def forward(self, pixel_values, grid_thw=None, plan=None, run=None):
        """Returns ``(merged [T/4, out], [deepstack features [T/4, out], ...])``."""
        run = run or (lambda m, *a, **k: m(*a, **k))
        plan = plan or self.plan(grid_thw, pixel_values.device)
        x = run(self.patch_embed, pixel_values, plan["pos_idx"], plan["pos_wt"])
        cos, sin = plan["cos"].to(x.dtype), plan["sin"].to(x.dtype)
        deep = []
        for i, blk in enumerate(self.blocks):
            x = run(blk, x, cos, sin, plan["cu_full"], plan["max_full"])
            if i in self.cfg.deepstack_visual_indexes:
                deep.append(run(self.deepstack_mergers[list(self.cfg.deepstack_visual_indexes).index(i)], x))
        return run(self.merger, x), deep


# ------------------------------------------------------------------------------------------ text decoder
class Qwen3DecoderLayer(nn.Module):
    """Pre-norm attention (per-head q/k RMSNorm, rotate-half RoPE, GQA) + dense SwiGLU or routed experts."""

    def __init__(self, c: Qwen3TextConfig, sparse: bool, num_local: Optional[int] = None):
        super().__init__()
        self.nq, self.nkv, self.hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.qkv_proj = Linear(c.hidden_size, (self.nq + 2 * self.nkv) * self.hd, bias=c.qkv_bias)
        self.o_proj = Linear(self.nq * self.hd, c.hidden_size, bias=False)
        self.q_norm = RMSNorm(self.hd, c.rms_norm_eps) if c.qk_norm else nn.Identity()
        self.k_norm = RMSNorm(self.hd, c.rms_norm_eps) if c.qk_norm else nn.Identity()
        self.sparse = sparse
        if sparse:
            self.mlp = SparseMoeBlock(c, num_local)
        else:
            self.gate_up_proj = Linear(c.hidden_size, 2 * c.intermediate_size, bias=False)
            self.down_proj = Linear(c.intermediate_size, c.hidden_size, bias=False)

    def _ffn(self, h, last: bool):
        if self.sparse:
            return self.mlp(h)
        return self.down_proj(ops.linear_swiglu(h, self.gate_up_proj.weight), value_unused_in_backward=last)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen, cache: Optional[dict] = None):
        T = x.shape[0]
        qkv = self.qkv_proj(self.input_layernorm(x))
        q, k, v = qkv.split([self.nq * self.hd, self.nkv * self.hd, self.nkv * self.hd], dim=-1)
        q = ops.rope_rotate_half(self.q_norm(q.reshape(T, self.nq, self.hd)), cos, sin)
        k = ops.rope_rotate_half(self.k_norm(k.reshape(T, self.nkv, self.hd)), cos, sin)
        v = v.reshape(T, self.nkv, self.hd)
        if cache is not None:                      # generation, one sequence: new tokens attend to all cached ones
            if "k" in cache:
                k, v = torch.cat([cache["k"], k]), torch.cat([cache["v"], v])
            cache["k"], cache["v"] = k, v
            L = k.shape[0]
            cu_q = torch.tensor([0, T], dtype=torch.int32, device=x.device)
            cu_k = torch.tensor([0, L], dtype=torch.int32, device=x.device)
            o = ops.attention_varlen(q, k, v, cu_q, cu_k, T, L, causal=True)
        else:
            o = ops.attention_varlen(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=True)
        x = x + self.o_proj(o.reshape(T, -1))
        return x + self._ffn(self.post_attention_layernorm(x), last=cache is None)


@model_register.register("qwen3_vl")
@model_register.register("qwen3_vl_moe")
@model_register.register("qwen3vl")            # the id the reference's transformers-backed trainer uses
class Qwen3VLModel(nn.Module):
    """Packed-sequence Qwen3-VL / Qwen3-VL-MoE for training and generation.

    ``forward(batch)`` takes the dict of the VLM collators (``input_ids`` [T], shifted ``labels`` [T], ``position_ids``
    [3, T], ``cu_seqlens``, ``max_seqlen``, optional ``pixel_values`` [P, 3 * 2 * 16 * 16] with ``image_grid_thw``) and
    returns ``(loss_sum, n_valid_tokens)``, or logits without labels.  With expert parallelism every rank holds
    ``num_experts / ep`` experts per layer."""

    def __init__(self, config: Qwen3VLConfig, ep_size: Optional[int] = None):
        super().__init__()
        self.config = config
        t = config.text
        ep = ep_size if ep_size is not None else get_parallel_state().size("ep")
        if t.num_experts and t.num_experts % ep:
            raise ValueError(f"num_experts {t.num_experts} must be divisible by expert_parallel_size {ep}")
        self.visual = Qwen3VisionTransformer(config.vision)
        self.embed_tokens = Embedding(t.vocab_size, t.hidden_size)
        self.layers = nn.ModuleList([
            Qwen3DecoderLayer(t, config.layer_is_sparse(i), t.num_experts // ep if t.num_experts else None)
            for i in range(t.num_layers)])
        self.lm_head = LMHead(t)
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

    # -- sharding plan -----------------------------------------------------------------------
    def fsdp_units(self) -> List[Tuple[str, nn.Module]]:
        v = self.visual
        units = [("embed_tokens", self.embed_tokens), ("visual.patch_embed", v.patch_embed)]
        units += [(f"visual.blocks.{i}", b) for i, b in enumerate(v.blocks)]
        units += [(f"visual.deepstack_mergers.{i}", m) for i, m in enumerate(v.deepstack_mergers)]
        units += [("visual.merger", v.merger)]
        units += [(f"layers.{i}", l) for i, l in enumerate(self.layers)]
        units += [("lm_head", self.lm_head)]
        return units

    def expert_units(self):
        """Expert parameter units (sharded over the expert-FSDP group, gradients divided by the world size)."""
        return [(f"layers.{i}.mlp.experts", l.mlp.experts) for i, l in enumerate(self.layers) if l.sparse]

    def hf_ops(self):
        """Hugging Face <-> internal name / layout operators (published checkpoint layout of the fused experts)."""
        from ..checkpoint.hf import qwen3vl_ops
        return qwen3vl_ops(self.config)

    def aux_loss(self):
        """Value of the router load-balancing term of the last forward (detached: its gradient is attached inside the
        MoE blocks, ``models/moe.py: _AttachAux``)."""
        ls = [l.mlp.aux_loss for l in self.layers if l.sparse and l.mlp.aux_loss is not None]
        return self.config.text.router_aux_loss_coef * torch.stack(ls).mean() if ls else None

    # -- forward -----------------------------------------------------------------------------
    def forward(self, batch: dict, run=None, kv_cache: Optional[list] = None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        t = self.config.text
        ids = batch["input_ids"]
        x = run(self.embed_tokens, ids)
        pv, deep, img_pos = batch.get("pixel_values"), [], None
        if pv is not None and pv.numel() > 0:
            plan = batch.get("vision_plan") or self.visual.plan(batch["image_grid_thw"], pv.device)
            v, deep = self.visual(pv.to(x.dtype), plan=plan, run=run)
            img_pos = batch.get("image_positions")
            if img_pos is None:
                img_pos = ((ids == self.config.image_token_id) | (ids == self.config.video_token_id)).nonzero(as_tuple=True)[0]
            x = x.index_copy(0, img_pos, v.to(x.dtype))
        cos, sin = batch.get("rope_cos"), batch.get("rope_sin")
        if cos is None:
            cos, sin = interleaved_mrope_cos_sin(batch["position_ids"], t.head_dim, t.rope_theta, t.mrope_section)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        for i, layer in enumerate(self.layers):
            if kv_cache is not None:
                x = run(layer, x, cos, sin, None, 0, kv_cache[i])
            else:
                x = run(layer, x, cos, sin, batch["cu_seqlens"], batch["max_seqlen"])
            if i < len(deep):                       # DeepStack: add the i-th vision feature at the visual positions
                x = x.index_add(0, img_pos, deep[i].to(x.dtype))
        if kv_cache is not None and batch.get("labels") is None:
            x = x[-1:]
        return run(self.lm_head, x, batch.get("labels"))
