"""Qwen2.5-VL (window-attention ViT + 2x2 merger + GQA/mRoPE decoder) on packed sequences.

Behavioural parity targets in the reference tree:
  * ViT, window index, 2-D rope: mindspeed_mm/models/vision/vision_encoders/qwen2vl_vit_model.py:329-530
  * merger:                      mindspeed_mm/models/vision/projectors/multimodal_projector.py:72-78
  * embedding scatter:           mindspeed_mm/models/vlm_model.py:545-556
  * mRoPE position ids:          mindspeed_mm/models/vision/vlm_attentionmask_for_llm.py:515-697
  * model dims:                  examples/qwen2.5vl/model_7b.json

The whole model runs in TND (packed, batch folded into T) layout: a micro-batch is one
stream of tokens plus ``cu_seqlens``; attention is varlen so samples never see each other.
QKV and gate/up projections are stored fused (one GEMM each); ``checkpoint/hf.py`` maps the
fused tensors to and from HuggingFace's per-projection names.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .registry import model_register


# --------------------------------------------------------------------------- configs
@dataclass
class VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    intermediate_size: int = 3420
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    window_size: int = 112
    fullatt_block_indexes: Sequence[int] = (7, 15, 23, 31)
    out_hidden_size: int = 3584
    rms_norm_eps: float = 1e-6
    tokens_per_second: int = 2


@dataclass
class TextConfig:
    num_layers: int = 28
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: Optional[int] = None
    vocab_size: int = 152064
    rope_theta: float = 1e6
    mrope_section: Sequence[int] = (16, 24, 24)
    rms_norm_eps: float = 1e-6
    qkv_bias: bool = True
    tie_word_embeddings: bool = False

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads


@dataclass
class Qwen25VLConfig:
    vision: VisionConfig = field(default_factory=VisionConfig)
    text: TextConfig = field(default_factory=TextConfig)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    init_std: float = 0.02

    @staticmethod
    def qwen2_5_vl_7b():
        return Qwen25VLConfig()

    @staticmethod
    def qwen2_5_vl_72b():
        return Qwen25VLConfig(
            vision=VisionConfig(out_hidden_size=8192),
            text=TextConfig(num_layers=80, hidden_size=8192, intermediate_size=29568,
                            num_attention_heads=64, num_key_value_heads=8))

    @staticmethod
    def tiny():
        """The CPU plumbing config: 4+4 layers, ViT 256, LLM 512, 8q/2kv, FFN 1376, vocab 32000."""
        return Qwen25VLConfig(
            vision=VisionConfig(depth=4, hidden_size=256, intermediate_size=688, num_heads=4,
                                fullatt_block_indexes=(1, 3), out_hidden_size=512),
            text=TextConfig(num_layers=4, hidden_size=512, intermediate_size=1376, num_attention_heads=8,
                            num_key_value_heads=2, vocab_size=32000, mrope_section=(8, 12, 12)),
            image_token_id=31999, video_token_id=31998, vision_start_token_id=31997)

    @staticmethod
    def from_mm_json(tree: dict) -> "Qwen25VLConfig":
        """Build from the ``--mm-model`` JSON tree (image_encoder / text_decoder)."""
        ve = tree["image_encoder"]["vision_encoder"]
        vp = tree["image_encoder"]["vision_projector"]
        td = tree["text_decoder"]
        vis = VisionConfig(
            depth=ve["num_layers"], hidden_size=ve["hidden_size"],
            intermediate_size=ve.get("intermediate_size", ve.get("ffn_hidden_size")),
            num_heads=ve["num_attention_heads"], in_channels=ve.get("in_channels", 3),
            patch_size=ve["patch_size"], temporal_patch_size=ve.get("temporal_patch_size", 2),
            spatial_merge_size=ve.get("spatial_merge_size", 2), window_size=ve.get("window_attn_size", 112),
            fullatt_block_indexes=tuple(ve.get("fullatt_block_indexes", ())),
            out_hidden_size=vp["hidden_size"], rms_norm_eps=ve.get("layernorm_epsilon", 1e-6),
            tokens_per_second=ve.get("tokens_per_second", 2))
        txt = TextConfig(
            num_layers=td["num_layers"], hidden_size=td["hidden_size"], intermediate_size=td["ffn_hidden_size"],
            num_attention_heads=td["num_attention_heads"],
            num_key_value_heads=td.get("num_query_groups", td["num_attention_heads"]),
            vocab_size=td["vocab_size"], rope_theta=td.get("rope_theta", 1e6),
            mrope_section=tuple(td.get("mrope_section", (16, 24, 24))),
            rms_norm_eps=td.get("layernorm_epsilon", 1e-6), qkv_bias=td.get("add_qkv_bias", True),
            tie_word_embeddings=not td.get("untie_embeddings_and_output_weights", True))
        return Qwen25VLConfig(vision=vis, text=txt, image_token_id=tree.get("img_context_token_id", 151655),
                              vision_start_token_id=tree.get("vision_start_token_id", 151652),
                              init_std=td.get("init_method_std", 0.02))


# --------------------------------------------------------------------------- index helpers (pure, CPU)
def vision_rot_pos_ids(grid_thw: torch.Tensor, merge: int) -> torch.Tensor:
    """(h, w) id of every patch in 2x2-merge order.  Returns [sum(t*h*w), 2] int64."""
    out = []
    for t, h, w in grid_thw.tolist():
        hp = torch.arange(h).unsqueeze(1).expand(-1, w)
        wp = torch.arange(w).unsqueeze(0).expand(h, -1)
        def blk(x):
            return x.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten()
        out.append(torch.stack([blk(hp), blk(wp)], dim=-1).repeat(t, 1))
    return torch.cat(out, 0)


def vision_window_index(grid_thw: torch.Tensor, window_size: int, merge: int, patch: int):
    """Window permutation of merged tokens and cumulative window lengths (in patch tokens).

    A window holds ``(window_size / merge / patch)^2`` merged tokens (4x4 for 112 px); the merged
    grid is padded to a multiple of that side, permuted to window-major order and the pads dropped.
    Returns (window_index [n_merged], cu_window_seqlens list[int] in units of patch tokens).
    """
    win = window_size // merge // patch
    unit = merge * merge
    window_index, cu = [], [0]
    base = 0
    for t, h, w in grid_thw.tolist():
        lh, lw = h // merge, w // merge
        idx = torch.arange(t * lh * lw).reshape(t, lh, lw)
        ph, pw = (-lh) % win, (-lw) % win
        nh, nw = (lh + ph) // win, (lw + pw) // win
        idx = F.pad(idx, (0, pw, 0, ph), value=-100)
        idx = idx.reshape(t, nh, win, nw, win).permute(0, 1, 3, 2, 4).reshape(t, nh * nw, win, win)
        seqlens = (idx != -100).sum([2, 3]).reshape(-1)
        flat = idx.reshape(-1)
        window_index.append(flat[flat != -100] + base)
        cs = seqlens.cumsum(0) * unit + cu[-1]
        cu.extend(cs.tolist())
        base += t * lh * lw
    # drop empty windows (consecutive duplicates)
    dedup = [cu[0]]
    for c in cu[1:]:
        if c != dedup[-1]:
            dedup.append(c)
    return torch.cat(window_index, 0), dedup


def get_rope_index(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], image_token_id: int,
                   vision_start_token_id: int, merge: int = 2,
                   second_per_grid_ts: Optional[Sequence[float]] = None, tokens_per_second: int = 2,
                   video_token_id: Optional[int] = None) -> Tuple[torch.Tensor, int]:
    """mRoPE (t, h, w) position ids for ONE sample.  input_ids: [S].  Returns ([3, S], delta).

    Text tokens advance all three axes together.  An image block of (t, h, w) merged tokens gets
    ``t*tokens_per_second*second_per_grid``, ``h`` and ``w`` offsets added to the running start;
    the text that follows restarts at ``max + 1``.
    """
    ids = input_ids.tolist()
    S = len(ids)
    pos = torch.zeros(3, S, dtype=torch.long)
    if image_grid_thw is None or len(image_grid_thw) == 0:
        pos[:] = torch.arange(S)
        return pos, 0
    grids = image_grid_thw.tolist()
    chunks, st, img_i, nxt = [], 0, 0, 0
    vis_ids = {image_token_id} | ({video_token_id} if video_token_id is not None else set())
    while st < S:
        # next vision token
        ed = st
        while ed < S and ids[ed] not in vis_ids:
            ed += 1
        if ed > st:
            n = ed - st
            chunks.append(torch.arange(n).view(1, -1).expand(3, -1) + nxt)
            nxt += n
        if ed >= S or img_i >= len(grids):
            if ed < S:  # vision tokens without a grid: treat as text
                n = S - ed
                chunks.append(torch.arange(n).view(1, -1).expand(3, -1) + nxt)
            break
        t, h, w = grids[img_i]
        is_video = video_token_id is not None and ids[ed] == video_token_id
        spg = (second_per_grid_ts[img_i] if (second_per_grid_ts is not None and is_video) else 0.0)
        img_i += 1
        lh, lw = h // merge, w // merge
        tt = (torch.arange(t).view(-1, 1).expand(-1, lh * lw) * spg * tokens_per_second).long().flatten()
        hh = torch.arange(lh).view(1, -1, 1).expand(t, -1, lw).flatten()
        ww = torch.arange(lw).view(1, 1, -1).expand(t, lh, -1).flatten()
        blk = torch.stack([tt, hh, ww]) + nxt
        chunks.append(blk)
        nxt = int(blk.max()) + 1
        st = ed + t * lh * lw
    pos = torch.cat(chunks, dim=1)[:, :S]
    return pos, int(pos.max()) + 1 - S


# --------------------------------------------------------------------------- layers
class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)


class Linear(nn.Module):
    """``nn.Linear`` twin whose forward goes through :func:`ops.linear`."""

    def __init__(self, in_features, out_features, bias=True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x, value_unused_in_backward: bool = False):
        return ops.linear(x, self.weight, self.bias, value_unused_in_backward)


class VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig):
        super().__init__()
        self.num_heads = c.num_heads
        self.head_dim = c.hidden_size // c.num_heads
        self.norm1 = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.norm2 = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.attn_qkv = Linear(c.hidden_size, 3 * c.hidden_size, bias=True)
        self.attn_proj = Linear(c.hidden_size, c.hidden_size, bias=True)
        # the FFN width is padded to a multiple of 64 (3420 -> 3456) so that every GEMM operand keeps
        # 16-byte aligned rows for TMA; the pad rows/columns are zero and contribute nothing
        self.ffn, self.ffn_padded = c.intermediate_size, (c.intermediate_size + 63) // 64 * 64
        self.mlp_gate_up = Linear(c.hidden_size, 2 * self.ffn_padded, bias=True)
        self.mlp_down = Linear(self.ffn_padded, c.hidden_size, bias=True)

    @torch.no_grad()
    def post_init(self):
        """Zero the padding of the FFN so the padded model computes exactly the unpadded one."""
        f, fp = self.ffn, self.ffn_padded
        if fp != f:
            for t in (self.mlp_gate_up.weight, self.mlp_gate_up.bias):
                t[f:fp].zero_()
                t[fp + f:].zero_()
            self.mlp_down.weight[:, f:].zero_()

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        T = x.shape[0]
        # one unbind (a single stack in backward) instead of three selects (three zero-filled adds in backward)
        q, k, v = self.attn_qkv(self.norm1(x)).view(T, 3, self.num_heads, self.head_dim).unbind(1)
        q = ops.rope_rotate_half(q, cos, sin)
        k = ops.rope_rotate_half(k, cos, sin)
        o = ops.attention_varlen(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=False)
        x = x + self.attn_proj(o.reshape(T, -1))
        # the block's last product only feeds the residual add: its value is not needed when the block is recomputed
        x = x + self.mlp_down(ops.swiglu(self.mlp_gate_up(self.norm2(x))), value_unused_in_backward=True)
        return x


class PatchMerger(nn.Module):
    def __init__(self, c: VisionConfig):
        super().__init__()
        self.unit = c.spatial_merge_size ** 2
        self.ln_q = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.fc1 = Linear(c.hidden_size * self.unit, c.hidden_size * self.unit)
        self.fc2 = Linear(c.hidden_size * self.unit, c.out_hidden_size)

    def forward(self, x):
        x = self.ln_q(x).view(-1, x.shape[-1] * self.unit)
        return self.fc2(ops.gelu(self.fc1(x)))


class VisionPatchEmbed(nn.Module):
    """Conv3d(kernel = stride = (tp, p, p)) applied to pre-flattened patches, i.e. one GEMM."""

    def __init__(self, c: VisionConfig):
        super().__init__()
        self.in_dim = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        self.proj = Linear(self.in_dim, c.hidden_size, bias=False)

    def forward(self, pixel_values):
        return self.proj(pixel_values.view(-1, self.in_dim))


class VisionTransformer(nn.Module):
    def __init__(self, c: VisionConfig):
        super().__init__()
        self.cfg = c
        self.patch_embed = VisionPatchEmbed(c)
        self.blocks = nn.ModuleList([VisionBlock(c) for _ in range(c.depth)])
        self.merger = PatchMerger(c)

    @torch.no_grad()
    def plan(self, grid_thw: torch.Tensor, device) -> dict:
        """All index tensors for a batch of images (host arithmetic; safe to precompute in the collator)."""
        c = self.cfg
        unit = c.spatial_merge_size ** 2
        head_dim = c.hidden_size // c.num_heads
        pos = vision_rot_pos_ids(grid_thw, c.spatial_merge_size)
        inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim // 2, 2, dtype=torch.float32) / (head_dim // 2)))
        freqs = (pos.unsqueeze(-1).float() * inv).flatten(1)          # [T, head_dim/2]
        emb = torch.cat((freqs, freqs), -1)                           # [T, head_dim]
        widx, cu_win = vision_window_index(grid_thw, c.window_size, c.spatial_merge_size, c.patch_size)
        T = pos.shape[0]
        perm = (widx.view(-1, 1) * unit + torch.arange(unit).view(1, -1)).flatten()   # patch-token permutation
        emb = emb[perm]
        lens = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])
        cu_full = F.pad(lens.cumsum(0), (1, 0)).to(torch.int32)
        cu_win_t = torch.tensor(cu_win, dtype=torch.int32)
        return dict(
            perm=perm.to(device), reverse=torch.argsort(widx).to(device),
            cos=emb.cos().to(device), sin=emb.sin().to(device),
            cu_full=cu_full.to(device), max_full=int(lens.max()),
            cu_win=cu_win_t.to(device), max_win=int((cu_win_t[1:] - cu_win_t[:-1]).max()), n_tokens=T)

    def embed(self, pixel_values, plan):
        x = self.patch_embed(pixel_values)
        return x.index_select(0, plan["perm"])

    def run_block(self, i, x, plan):
        full = i in self.cfg.fullatt_block_indexes
        cu, mx = (plan["cu_full"], plan["max_full"]) if full else (plan["cu_win"], plan["max_win"])
        return self.blocks[i](x, plan["cos"].to(x.dtype), plan["sin"].to(x.dtype), cu, mx)

    def finish(self, x, plan):
        return self.merger(x).index_select(0, plan["reverse"])

    def forward(self, pixel_values, grid_thw=None, plan=None):
        plan = plan or self.plan(grid_thw, pixel_values.device)
        x = self.embed(pixel_values, plan)
        for i in range(len(self.blocks)):
            x = self.run_block(i, x, plan)
        return self.finish(x, plan)


class DecoderLayer(nn.Module):
    def __init__(self, c: TextConfig):
        super().__init__()
        self.nq, self.nkv, self.hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.qkv_proj = Linear(c.hidden_size, (self.nq + 2 * self.nkv) * self.hd, bias=c.qkv_bias)
        self.o_proj = Linear(self.nq * self.hd, c.hidden_size, bias=False)
        self.gate_up_proj = Linear(c.hidden_size, 2 * c.intermediate_size, bias=False)
        self.down_proj = Linear(c.intermediate_size, c.hidden_size, bias=False)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen, cache: Optional[dict] = None):
        """``cache`` (generation, one sequence): a dict that keeps this layer's rotated keys and the values of all
        tokens seen so far; the new tokens attend to them (causal mask aligned to the end of the key sequence)."""
        T = x.shape[0]
        qkv = self.qkv_proj(self.input_layernorm(x))
        q, k, v = qkv.split([self.nq * self.hd, self.nkv * self.hd, self.nkv * self.hd], dim=-1)
        q = ops.rope_rotate_half(q.view(T, self.nq, self.hd), cos, sin)
        k = ops.rope_rotate_half(k.view(T, self.nkv, self.hd), cos, sin)
        v = v.view(T, self.nkv, self.hd)
        if cache is not None:
            if "k" in cache:
                k, v = torch.cat([cache["k"], k]), torch.cat([cache["v"], v])
            cache["k"], cache["v"] = k, v
            L = k.shape[0]
            cu_q = torch.tensor([0, T], dtype=torch.int32, device=x.device)
            cu_k = torch.tensor([0, L], dtype=torch.int32, device=x.device)
            o = ops.attention_varlen(q, k, v, cu_q, cu_k, T, L, causal=True)
            x = x + self.o_proj(o.reshape(T, -1))
            return x + self.down_proj(ops.linear_swiglu(self.post_attention_layernorm(x), self.gate_up_proj.weight))
        o = ops.attention_varlen(q, k, v, cu_seqlens, cu_seqlens,
                                 max_seqlen, max_seqlen, causal=True)
        x = x + self.o_proj(o.reshape(T, -1))
        x = x + self.down_proj(ops.linear_swiglu(self.post_attention_layernorm(x), self.gate_up_proj.weight),
                               value_unused_in_backward=True)
        return x


class LMHead(nn.Module):
    """Final norm + vocabulary projection + cross entropy, fused so [T, V] logits never exist."""

    def __init__(self, c: TextConfig):
        super().__init__()
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.weight = nn.Parameter(torch.empty(c.vocab_size, c.hidden_size))

    def forward(self, x, labels=None, prenormed: bool = False, norm_only: bool = False):
        """``prenormed``: ``x`` already went through a final norm of its own (multi-token-prediction block);
        ``norm_only``: return the normalised hidden states instead of logits / loss."""
        h = x if prenormed else self.norm(x)
        if norm_only:
            return h
        if labels is None:
            return ops.linear(h, self.weight)
        return ops.linear_cross_entropy(h, self.weight, labels)


class Embedding(nn.Module):
    def __init__(self, vocab, dim):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim))

    def forward(self, ids):
        return F.embedding(ids, self.weight)


@model_register.register("qwen2_5vl")
class Qwen25VLModel(nn.Module):
    """Packed-sequence Qwen2.5-VL for training.

    ``forward(batch)`` takes the dict produced by the VLM collators:
      input_ids [T] int64, labels [T] int64 (already shifted; -100 = ignored), position_ids [3, T],
      cu_seqlens [n+1] int32, max_seqlen int, pixel_values [P, 1176] (optional), image_grid_thw [n_img, 3] (CPU).
    and returns ``(loss_sum, n_valid_tokens)``; the loss function decides the normalisation.
    """

    def __init__(self, config: Qwen25VLConfig):
        super().__init__()
        self.config = config
        t = config.text
        self.visual = VisionTransformer(config.vision)
        self.embed_tokens = Embedding(t.vocab_size, t.hidden_size)
        self.layers = nn.ModuleList([DecoderLayer(t) for _ in range(t.num_layers)])
        self.lm_head = LMHead(t)
        # parallel.data_balance.EncoderBalance over the data-parallel group (``--encoder-dp-balance``): images are
        # re-dealt across ranks before the vision tower and their embeddings sent back after it
        self.encoder_balance = None

    # -- init ------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        std = self.config.init_std
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                # draw on CPU in fp32 chunks so every world size / device sees the same values
                p.copy_(_normal_like(p, std, g))
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)

    # -- FSDP plan -------------------------------------------------------------------------
    def fsdp_units(self) -> List[Tuple[str, nn.Module]]:
        """Modules that are sharded/gathered as one unit, in execution order."""
        units = [("embed_tokens", self.embed_tokens), ("visual.patch_embed", self.visual.patch_embed)]
        units += [(f"visual.blocks.{i}", b) for i, b in enumerate(self.visual.blocks)]
        units += [("visual.merger", self.visual.merger)]
        units += [(f"layers.{i}", l) for i, l in enumerate(self.layers)]
        units += [("lm_head", self.lm_head)]
        return units

    # -- forward ---------------------------------------------------------------------------
    def forward(self, batch: dict, run=None, kv_cache: Optional[list] = None):
        """``run(module, *args)`` lets the parallel engine wrap each unit (gather/recompute/reduce).
        ``kv_cache`` (generation): one dict per decoder layer, filled by the prefill call and extended by every later
        call, whose ``batch`` then holds only the new tokens (``input_ids`` / ``position_ids`` of those, no pixels)."""
        run = run or (lambda m, *a, **k: m(*a, **k))
        t = self.config.text
        ids = batch["input_ids"]
        x = run(self.embed_tokens, ids)
        pv = batch.get("pixel_values")
        if pv is not None and pv.numel() > 0:
            vis = self.visual
            book = None
            if self.encoder_balance is not None:
                grid = batch["image_grid_thw"]
                pv, book = self.encoder_balance.dispatch(pv, grid.prod(-1).tolist(), grid.tolist())
            if book is not None:
                plan = vis.plan(book["grids"], pv.device)
            else:
                plan = batch.get("vision_plan") or vis.plan(batch["image_grid_thw"], pv.device)
            v = run(vis.patch_embed, pv.to(x.dtype)).index_select(0, plan["perm"])
            for i in range(len(vis.blocks)):
                full = i in vis.cfg.fullatt_block_indexes
                cu, mx = (plan["cu_full"], plan["max_full"]) if full else (plan["cu_win"], plan["max_win"])
                v = run(vis.blocks[i], v, plan["cos"].to(x.dtype), plan["sin"].to(x.dtype), cu, mx)
            v = run(vis.merger, v).index_select(0, plan["reverse"])
            if book is not None:
                v = self.encoder_balance.combine(v, book, ratio=vis.cfg.spatial_merge_size ** 2)
            img_pos = batch.get("image_positions")
            if img_pos is None:
                img_pos = (ids == self.config.image_token_id).nonzero(as_tuple=True)[0]
            x = x.index_copy(0, img_pos, v.to(x.dtype))
        cos, sin = batch.get("rope_cos"), batch.get("rope_sin")
        if cos is None:
            cos, sin = ops.ref.mrope_cos_sin(batch["position_ids"], t.head_dim, t.rope_theta, t.mrope_section)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        for i, layer in enumerate(self.layers):
            if kv_cache is not None:
                x = run(layer, x, cos, sin, None, 0, kv_cache[i])
            else:
                x = run(layer, x, cos, sin, batch["cu_seqlens"], batch["max_seqlen"])
        if kv_cache is not None and batch.get("labels") is None:
            x = x[-1:]                      # generation reads the last position only
        return run(self.lm_head, x, batch.get("labels"))


def _normal_like(p: torch.Tensor, std: float, g: torch.Generator) -> torch.Tensor:
    out = torch.empty(p.shape, dtype=torch.float32)
    out.normal_(0.0, std, generator=g)
    return out.to(device=p.device, dtype=p.dtype)
