"""InternVL data path: dynamic tiling of images into 448 x 448 tiles, ``<img><IMG_CONTEXT>...</img>`` prompts, and a
collator that packs samples for ``models/internvl.py``.

Reference: mindspeed_mm/data/data_utils/multimodal_image_video_preprocess.py (``dynamic_preprocess`` :137,
``find_closest_aspect_ratio`` :117, ``InternvlImageVideoPreprocess`` :67) and the ``internvl`` collator of
mindspeed_mm/data/dataloader/data_collator.py.  An image is resized to the tile grid (columns x rows, ``min_tiles <=
columns * rows <= max_tiles``) whose aspect ratio is closest to its own; on ties the larger grid wins when the image has
more than half the grid's pixels.  With more than one tile a thumbnail of the whole image follows as the last tile.
Every tile yields ``(image_size / patch * downsample)^2`` placeholder tokens.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..models.registry import data_register
from .collate import pin_batch
from .multimodal import MultimodalConversationDataset

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


def tile_grids(min_tiles: int, max_tiles: int) -> List[Tuple[int, int]]:
    """All (columns, rows) with ``min_tiles <= columns * rows <= max_tiles``, smaller grids first."""
    grids = {(c, r) for c in range(1, max_tiles + 1) for r in range(1, max_tiles + 1) if min_tiles <= c * r <= max_tiles}
    return sorted(grids, key=lambda g: (g[0] * g[1], g))


def closest_tile_grid(width: int, height: int, grids: Sequence[Tuple[int, int]], image_size: int) -> Tuple[int, int]:
    aspect, best, best_diff = width / height, (1, 1), float("inf")
    for c, r in grids:
        diff = abs(aspect - c / r)
        if diff < best_diff:
            best, best_diff = (c, r), diff
        elif diff == best_diff and width * height > 0.5 * image_size * image_size * c * r:
            best = (c, r)
    return best


class InternVLTileProcessor:
    """Image -> normalised tiles ``[n, 3, S, S]`` and a pseudo grid ``(n, 1, tokens_per_tile)`` whose product is the
    number of placeholder tokens (the shape contract of the conversation dataset's image processors)."""

    merge = 1

    def __init__(self, image_size: int = 448, patch_size: int = 14, downsample_ratio: float = 0.5, min_tiles: int = 1,
                 max_tiles: int = 12, use_thumbnail: bool = True, dynamic: bool = True,
                 mean: Sequence[float] = IMAGENET_MEAN, std: Sequence[float] = IMAGENET_STD):
        self.size, self.patch, self.ratio = image_size, patch_size, downsample_ratio
        self.grids = tile_grids(min_tiles, max_tiles) if dynamic else [(1, 1)]
        self.use_thumbnail = use_thumbnail
        self.tokens_per_tile = int(image_size // patch_size * downsample_ratio) ** 2
        self.mean = torch.tensor(mean).view(1, 3, 1, 1)
        self.std = torch.tensor(std).view(1, 3, 1, 1)

    @classmethod
    def for_config(cls, cfg, **kw) -> "InternVLTileProcessor":
        return cls(image_size=cfg.vision.image_size, patch_size=cfg.vision.patch_size,
                   downsample_ratio=cfg.downsample_ratio, **kw)

    @staticmethod
    def _to_tensor(img) -> torch.Tensor:
        if isinstance(img, torch.Tensor):
            t = img.float() / 255.0 if img.dtype == torch.uint8 else img
            return t if t.shape[0] == 3 else t.permute(2, 0, 1)
        import numpy as np
        arr = np.asarray(img.convert("RGB") if hasattr(img, "convert") else img)
        return torch.from_numpy(arr.copy()).permute(2, 0, 1).float() / 255.0

    def _resize(self, t: torch.Tensor, h: int, w: int) -> torch.Tensor:
        return F.interpolate(t[None], size=(h, w), mode="bicubic", align_corners=False, antialias=True)[0].clamp(0, 1)

    def tiles(self, img) -> torch.Tensor:
        t = self._to_tensor(img)
        S = self.size
        c, r = closest_tile_grid(t.shape[2], t.shape[1], self.grids, S)
        big = self._resize(t, r * S, c * S)
        out = big.view(3, r, S, c, S).permute(1, 3, 0, 2, 4).reshape(r * c, 3, S, S)       # row by row
        if self.use_thumbnail and r * c > 1:
            out = torch.cat([out, self._resize(t, S, S)[None]])
        return (out - self.mean) / self.std

    def __call__(self, img):
        x = self.tiles(img)
        return x, (x.shape[0], 1, self.tokens_per_tile)

    def frames(self, frames: torch.Tensor):
        """Video frames [T, 3, H, W] in [0, 1]: one tile per frame."""
        x = F.interpolate(frames, size=(self.size, self.size), mode="bicubic", align_corners=False, antialias=True)
        x = (x.clamp(0, 1) - self.mean) / self.std
        return x, (x.shape[0], 1, self.tokens_per_tile)

    def empty(self) -> torch.Tensor:
        return torch.zeros(0, 3, self.size, self.size)


@data_register.register("internvl")
class InternVLConversationDataset(MultimodalConversationDataset):
    """Conversation records (``messages`` / ShareGPT ``conversations`` with ``<image>`` / ``<video>`` marks) -> token
    ids with ``<img>`` + placeholders + ``</img>`` per image, supervised-span labels, and the image tiles.  Dataset keys
    of the reference's recipe are read from ``dataset_param`` (``image_size``, ``patch_size``, ``down_sample_ratio``,
    ``dynamic_image_size``, ``use_thumbnail``, ``min_dynamic_patch``, ``max_dynamic_patch``, ``template_name``)."""

    def __init__(self, dataset_param=None, model=None, *, processor: Optional[InternVLTileProcessor] = None, **kw):
        cfg = getattr(model, "config", None)
        if processor is None:
            extra = dict(getattr(dataset_param, "model_extra", None) or {}) if dataset_param is not None else {}
            basic = dict(getattr(dataset_param, "basic_parameters", None) or {}) if dataset_param is not None else {}
            get = lambda k, d: extra.get(k, basic.get(k, d))
            processor = InternVLTileProcessor(
                image_size=int(get("image_size", cfg.vision.image_size if cfg else 448)),
                patch_size=int(get("patch_size", cfg.vision.patch_size if cfg else 14)),
                downsample_ratio=float(get("down_sample_ratio", cfg.downsample_ratio if cfg else 0.5)),
                min_tiles=int(get("min_dynamic_patch", 1)), max_tiles=int(get("max_dynamic_patch", 12)),
                use_thumbnail=bool(get("use_thumbnail", True)), dynamic=bool(get("dynamic_image_size", True)))
        if kw.get("template") is None:
            import os
            from .multimodal import ByteTokenizer
            from .templates import TEMPLATES, TemplateRenderer
            pre = dict(getattr(dataset_param, "preprocess_parameters", None) or {}) if dataset_param is not None else {}
            extra = dict(getattr(dataset_param, "model_extra", None) or {}) if dataset_param is not None else {}
            tok = kw.get("tokenizer")
            path = pre.get("model_name_or_path") or (extra.get("tokenizer_config") or {}).get("from_pretrained")
            if tok is None and path and os.path.exists(path):
                from transformers import AutoTokenizer
                tok = AutoTokenizer.from_pretrained(path)
            name = pre.get("template") or pre.get("template_name") or extra.get("template_name") or "internvl"
            if name not in TEMPLATES:
                raise ValueError(f"Template {name} does not exist (known: {sorted(TEMPLATES)})")
            media = None
            if tok is None:              # stand-in byte tokenizer: the placeholder ids are the model's
                tok = ByteTokenizer()
                trio = (getattr(cfg, "vision_start_token_id", None), cfg.image_token_id,
                        getattr(cfg, "vision_end_token_id", None))
                media = {"image": trio, "video": trio}
            kw["tokenizer"], kw["template"] = tok, TemplateRenderer(TEMPLATES[name], tok, media_ids=media)
        super().__init__(dataset_param, model, processor=processor, **kw)


class TilePackCollator:
    """Packs tile samples into one token stream: next-token labels inside each sample, ``cu_seqlens``, all tiles in
    order, and the positions of the placeholder tokens."""

    def __init__(self, image_token_id: int, ignore_index: int = -100, pixel_dtype: torch.dtype = torch.float32,
                 pin: bool = False):
        self.image_token_id, self.ignore_index, self.pixel_dtype, self.pin = image_token_id, ignore_index, pixel_dtype, pin

    @classmethod
    def for_config(cls, cfg, **kw) -> "TilePackCollator":
        return cls(cfg.image_token_id, **kw)

    def __call__(self, samples: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        ids, labels, lens, pix = [], [], [], []
        for s in samples:
            i, l = s["input_ids"], s["labels"]
            ids.append(i)
            labels.append(torch.cat([l[1:], l.new_full((1,), self.ignore_index)]))
            lens.append(len(i))
            pv = s.get("pixel_values")
            if pv is not None and pv.shape[0]:
                pix.append(pv)
        input_ids = torch.cat(ids)
        out = dict(input_ids=input_ids, labels=torch.cat(labels),
                   cu_seqlens=F.pad(torch.tensor(lens).cumsum(0), (1, 0)).to(torch.int32), max_seqlen=max(lens),
                   n_tokens=int(input_ids.numel()))
        if pix:
            out["pixel_values"] = torch.cat(pix).to(self.pixel_dtype)
            out["image_positions"] = (input_ids == self.image_token_id).nonzero(as_tuple=True)[0]
        return pin_batch(out) if self.pin else out
