"""Packing collator for VLM samples.

Takes a list of samples (``input_ids``, ``labels``, ``pixel_values``, ``image_grid_thw``) and emits ONE
packed TND micro-batch: ids/labels concatenated to [T], next-token labels already shifted inside
each sample (the token after a sample's last one is never a target), ``cu_seqlens`` for varlen
attention, per-sample mRoPE position ids, the flat patch matrix and the ViT index plan.

Reference behaviour: DynamicBatchingDataLoader + batching strategy
(mindspeed_mm/data/dataloader/dynamic_batching_dataloader.py:37-159, batching_strategy.py:16-130)
and the Qwen2-VL collator that masks image tokens (mindspeed_mm/data/dataloader/data_collator.py:182-197).
Everything here is host arithmetic on CPU tensors; ``to_device`` does the one H2D hop.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..models.qwen2_5_vl import get_rope_index, vision_rot_pos_ids, vision_window_index


class PackedVLMCollator:
    def __init__(self, image_token_id: int, vision_start_token_id: int, merge: int = 2, patch: int = 14,
                 window_size: int = 112, vit_head_dim: int = 80, ignore_index: int = -100,
                 pad_to: Optional[int] = None, pixel_dtype: torch.dtype = torch.float32, pin: bool = False,
                 rope_index_fn=None, vision_plan_fn=None):
        self.image_token_id, self.vision_start_token_id = image_token_id, vision_start_token_id
        self.merge, self.patch, self.window_size, self.vit_head_dim = merge, patch, window_size, vit_head_dim
        self.ignore_index, self.pad_to, self.pixel_dtype, self.pin = ignore_index, pad_to, pixel_dtype, pin
        # model families whose position ids / vision index plan differ from Qwen2.5-VL's hand theirs over
        self.rope_index_fn = rope_index_fn or (
            lambda i, g: get_rope_index(i, g, self.image_token_id, self.vision_start_token_id, self.merge))
        self.vision_plan_fn = vision_plan_fn or (
            lambda grid: vision_plan(grid, self.merge, self.patch, self.window_size, self.vit_head_dim))

    @classmethod
    def for_config(cls, cfg, **kw) -> "PackedVLMCollator":
        """Collator for a VLM config (``image_token_id``, ``vision``): a config that defines ``rope_index`` /
        ``vision_plan`` (Qwen3-VL) supplies its own position ids and vision plan."""
        v = getattr(cfg, "vision", None)
        if v is None:                       # the composable model's plain ViT, or no tower at all
            v = getattr(cfg, "vit", None)
            merge = getattr(v, "merge", 2)
            return cls(cfg.image_token_id, cfg.vision_start_token_id, merge=merge, patch=getattr(v, "patch_size", 14),
                       vision_plan_fn=lambda grid: None, **kw)
        if not hasattr(v, "spatial_merge_size"):          # a tower of another family (wrapped transformers classes): no plan
            return cls(cfg.image_token_id, cfg.vision_start_token_id, merge=getattr(cfg, "spatial_merge_size", 2) or 2,
                       patch=getattr(v, "patch_size", 14), vision_plan_fn=lambda grid: None, **kw)
        return cls(cfg.image_token_id, cfg.vision_start_token_id, merge=v.spatial_merge_size, patch=v.patch_size,
                   window_size=getattr(v, "window_size", 0), vit_head_dim=v.hidden_size // v.num_heads,
                   rope_index_fn=getattr(cfg, "rope_index", None), vision_plan_fn=getattr(cfg, "vision_plan", None), **kw)

    def __call__(self, samples: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        ids, labels, pos, lens, pix, grids = [], [], [], [], [], []
        for s in samples:
            i = s["input_ids"]
            l = s["labels"]
            shifted = torch.cat([l[1:], l.new_full((1,), self.ignore_index)])
            g = s.get("image_grid_thw")
            p, _ = self.rope_index_fn(i, g)
            ids.append(i); labels.append(shifted); pos.append(p); lens.append(len(i))
            if g is not None and len(g):
                pix.append(s["pixel_values"]); grids.append(g)
        input_ids = torch.cat(ids)
        out = dict(
            input_ids=input_ids, labels=torch.cat(labels), position_ids=torch.cat(pos, dim=1),
            cu_seqlens=F.pad(torch.tensor(lens).cumsum(0), (1, 0)).to(torch.int32), max_seqlen=max(lens),
            n_tokens=int(input_ids.numel()))
        if pix:
            grid = torch.cat(grids)
            out["pixel_values"] = torch.cat(pix).to(self.pixel_dtype)
            out["image_grid_thw"] = grid
            out["image_positions"] = (input_ids == self.image_token_id).nonzero(as_tuple=True)[0]
            out["vision_plan"] = self.vision_plan_fn(grid)
        if self.pin:
            out = pin_batch(out)
        return out


def vision_plan(grid_thw: torch.Tensor, merge: int, patch: int, window_size: int, head_dim: int) -> dict:
    """CPU twin of ``VisionTransformer.plan``: permutation, 2-D rope tables and both cu_seqlens."""
    unit = merge * merge
    pos = vision_rot_pos_ids(grid_thw, merge)
    inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim // 2, 2, dtype=torch.float32) / (head_dim // 2)))
    freqs = (pos.unsqueeze(-1).float() * inv).flatten(1)
    emb = torch.cat((freqs, freqs), -1)
    widx, cu_win = vision_window_index(grid_thw, window_size, merge, patch)
    perm = (widx.view(-1, 1) * unit + torch.arange(unit).view(1, -1)).flatten()
    emb = emb[perm]
    lens = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])
    cu_win_t = torch.tensor(cu_win, dtype=torch.int32)
    return dict(perm=perm, reverse=torch.argsort(widx), cos=emb.cos(), sin=emb.sin(),
                cu_full=F.pad(lens.cumsum(0), (1, 0)).to(torch.int32), max_full=int(lens.max()),
                cu_win=cu_win_t, max_win=int((cu_win_t[1:] - cu_win_t[:-1]).max()), n_tokens=int(pos.shape[0]))


def _map(obj, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, dict):
        return {k: _map(v, fn) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_map(v, fn) for v in obj)
    return obj


def pin_batch(batch):
    return _map(batch, lambda t: t.pin_memory() if torch.cuda.is_available() else t)


HOST_KEYS = ("image_grid_thw",)


def to_device(batch: dict, device, non_blocking: bool = True) -> dict:
    """One H2D hop for every tensor except the few that only host code reads."""
    out = {}
    for k, v in batch.items():
        out[k] = v if k in HOST_KEYS else _map(v, lambda t: t.to(device, non_blocking=non_blocking))
    return out


def batch_nbytes(batch) -> int:
    n = 0
    def acc(t):
        nonlocal n
        n += t.numel() * t.element_size()
        return t
    _map({k: v for k, v in batch.items() if k not in HOST_KEYS}, acc)
    return n
