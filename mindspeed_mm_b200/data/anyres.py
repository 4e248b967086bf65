"""Any-resolution image tiling for tile-based VLMs (DeepSeek-VL2, LLaVA-NeXT style).

An image becomes one *global view* (the whole picture padded to a square of ``image_size``) plus a grid of
``tiles_w x tiles_h`` *local views* cut from the picture padded to the best fitting candidate resolution.  The prompt gets
``h * (w + 1)`` placeholder tokens for the global view (one extra per row for a line-break embedding), one separator and
``(tiles_h * h) * (tiles_w * w + 1)`` tokens for the local grid, where ``h = w = ceil(image_size / patch / downsample)``.

Reference: mindspeed_mm/data/data_utils/processing_deepseek_vl_v2.py (``select_best_resolution`` :35,
``tokenize_with_images`` :542-612, ``process_one`` :381); the model side that lays the tile features out in this order is
``models/composable.py: TileFormatter`` (mindspeed_mm/models/deepseekvl_model.py:313-428).  Images are float tensors
``[3, H, W]`` in [0, 1] here (PIL images are converted), so the whole path runs without an image library.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Sequence, Tuple

import torch
import torch.nn.functional as F


def candidate_grid(image_size: int, max_tiles: int = 9, min_tiles: int = 1) -> List[Tuple[int, int]]:
    """All (width, height) that are whole multiples of ``image_size`` with ``min_tiles <= tiles <= max_tiles``."""
    out = []
    for tw in range(1, max_tiles + 1):
        for th in range(1, max_tiles + 1):
            if min_tiles <= tw * th <= max_tiles:
                out.append((tw * image_size, th * image_size))
    return out


def select_best_resolution(image_size: Sequence[int], candidates: Sequence[Sequence[int]]) -> Tuple[int, int]:
    """(width, height) of the candidate that keeps most of the picture's pixels after an aspect-preserving fit, ties broken
    by the least padding.  ``image_size`` is (width, height)."""
    ow, oh = image_size
    best, best_eff, best_waste = None, 0, float("inf")
    for w, h in candidates:
        s = min(w / ow, h / oh)
        eff = min(int(ow * s) * int(oh * s), ow * oh)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (w, h), eff, waste
    return best


def to_tensor(img) -> torch.Tensor:
    """PIL image / uint8 array / float tensor -> float32 [3, H, W] in [0, 1]."""
    if isinstance(img, torch.Tensor):
        t = img
    else:
        import numpy as np
        a = np.asarray(img.convert("RGB") if hasattr(img, "convert") else img)
        t = torch.from_numpy(a.copy()).permute(2, 0, 1)
    if t.dtype == torch.uint8:
        t = t.float() / 255.0
    return t.float()


def fit_and_pad(img: torch.Tensor, size: Tuple[int, int], fill: Sequence[float]) -> torch.Tensor:
    """Resize ``img`` [3, H, W] to fit inside (width, height) keeping its aspect, centred on a canvas of ``fill`` colour."""
    W, H = size
    _, h, w = img.shape
    s = min(W / w, H / h)
    nw, nh = max(1, min(W, round(w * s))), max(1, min(H, round(h * s)))
    if (nh, nw) != (h, w):
        img = F.interpolate(img[None], size=(nh, nw), mode="bicubic", align_corners=False, antialias=True)[0].clamp(0, 1)
    canvas = torch.tensor(list(fill), dtype=img.dtype).view(3, 1, 1).expand(3, H, W).clone()
    top, left = (H - nh) // 2, (W - nw) // 2
    canvas[:, top:top + nh, left:left + nw] = img
    return canvas


@dataclass
class AnyResSpec:
    image_size: int = 384
    patch_size: int = 16
    downsample_ratio: int = 2
    candidates: Sequence[Sequence[int]] = field(default_factory=lambda: candidate_grid(384, 9))
    mean: Sequence[float] = (0.5, 0.5, 0.5)
    std: Sequence[float] = (0.5, 0.5, 0.5)
    image_token: str = "<image>"
    image_token_id: int = 100003
    ignore_id: int = -100

    @property
    def tokens_per_side(self) -> int:
        return math.ceil(self.image_size // self.patch_size / self.downsample_ratio)


def image_token_count(spec: AnyResSpec, tiles_w: int, tiles_h: int) -> int:
    h = w = spec.tokens_per_side
    return h * (w + 1) + 1 + (tiles_h * h) * (tiles_w * w + 1)


def tile_views(img, spec: AnyResSpec, cropping: bool = True) -> Tuple[torch.Tensor, Tuple[int, int]]:
    """-> (views [1 + tiles_w * tiles_h, 3, S, S] normalised, (tiles_w, tiles_h)); view 0 is the global one, local views
    follow row by row."""
    t = to_tensor(img)
    S = spec.image_size
    bw, bh = select_best_resolution((t.shape[2], t.shape[1]), spec.candidates) if cropping else (S, S)
    mean = torch.tensor(list(spec.mean)).view(3, 1, 1)
    std = torch.tensor(list(spec.std)).view(3, 1, 1)
    views = [fit_and_pad(t, (S, S), spec.mean)]
    local = fit_and_pad(t, (bw, bh), spec.mean)
    for i in range(0, bh, S):
        for j in range(0, bw, S):
            views.append(local[:, i:i + S, j:j + S])
    return (torch.stack(views) - mean) / std, (bw // S, bh // S)


def tokenize_with_images(text: str, images: Sequence, encode: Callable[[str], List[int]], spec: AnyResSpec,
                         bos_id: int = None, eos_id: int = None, cropping: bool = True):
    """Split ``text`` at the image tag, encode the pieces and put each image's placeholder run between them.

    Returns ``dict(input_ids, images_seq_mask, views [n_views, 3, S, S], spatial_crop [n_images, 2] as (tiles_w, tiles_h),
    num_image_tokens)``."""
    parts = text.split(spec.image_token)
    if len(parts) - 1 != len(images):
        raise ValueError(f"{len(parts) - 1} image tags in the text but {len(images)} images")
    ids: List[int] = []
    mask: List[bool] = []
    views, crops, counts = [], [], []
    for piece, img in zip(parts, images):
        enc = encode(piece)
        ids += enc
        mask += [False] * len(enc)
        v, (tw, th) = tile_views(img, spec, cropping)
        views.append(v)
        crops.append([tw, th])
        n = image_token_count(spec, tw, th)
        ids += [spec.image_token_id] * n
        mask += [True] * n
        counts.append(n)
    enc = encode(parts[-1])
    ids += enc
    mask += [False] * len(enc)
    if bos_id is not None:
        ids, mask = [bos_id] + ids, [False] + mask
    if eos_id is not None:
        ids, mask = ids + [eos_id], mask + [False]
    S = spec.image_size
    return dict(input_ids=torch.tensor(ids, dtype=torch.long), images_seq_mask=torch.tensor(mask, dtype=torch.bool),
                views=torch.cat(views) if views else torch.zeros(0, 3, S, S),
                spatial_crop=torch.tensor(crops, dtype=torch.long).view(-1, 2), num_image_tokens=counts)


def build_sft_sample(turns: Sequence[Tuple[str, str]], images: Sequence, encode: Callable[[str], List[int]],
                     spec: AnyResSpec, bos_id: int = None, eos_id: int = None, role_tags=("<|User|>: ", "<|Assistant|>: "),
                     sep: str = "\n\n") -> dict:
    """Chat turns ``[(user_text, assistant_text), ...]`` -> one training sample: labels cover the assistant replies (and the
    end token), everything else -- prompts and image placeholders -- is ignored by the loss."""
    ids: List[torch.Tensor] = []
    labels: List[torch.Tensor] = []
    masks: List[torch.Tensor] = []
    views, crops = [], []
    it = iter(images)
    for n, (user, reply) in enumerate(turns):
        want = user.count(spec.image_token)
        q = tokenize_with_images(role_tags[0] + user + sep + role_tags[1], [next(it) for _ in range(want)], encode, spec,
                                 bos_id=bos_id if n == 0 else None)
        a = torch.tensor(encode(reply) + ([eos_id] if eos_id is not None else []), dtype=torch.long)
        ids += [q["input_ids"], a]
        labels += [torch.full_like(q["input_ids"], spec.ignore_id), a.clone()]
        masks += [q["images_seq_mask"], torch.zeros_like(a, dtype=torch.bool)]
        views.append(q["views"])
        crops.append(q["spatial_crop"])
    return dict(input_ids=torch.cat(ids), labels=torch.cat(labels), images_seq_mask=torch.cat(masks),
                views=torch.cat(views), spatial_crop=torch.cat(crops))


def views_to_patch_rows(views: torch.Tensor, patch: int, merge: int = 2, temporal: int = 1):
    """Normalised views [n, 3, S, S] -> (patch rows [n * (S/p)^2, 3 * temporal * p * p] in merge-group order,
    grid_thw [n, 3]): the layout the plain ViT tower reads."""
    n, C, H, W = views.shape
    gh, gw = H // patch, W // patch
    x = views[:, None].expand(n, temporal, C, H, W).reshape(n, temporal, C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(n * gh * gw, C * temporal * patch * patch)
    grid = torch.tensor([[1, gh, gw]] * n, dtype=torch.long).view(-1, 3)
    return x, grid


# ------------------------------------------------------------------------------------------------- dataset + collator
class TiledConversationDataset(torch.utils.data.Dataset):
    """ShareGPT / messages records with ``<image>`` tags -> tiled SFT samples (``build_sft_sample``).  Registered as
    ``deepseekvl2`` (mindspeed_mm/data/datasets/deepseekvl2_dataset.py builds the same fields through the processor's
    ``process_one``).  ``image_loader(path) -> PIL image or [3, H, W] tensor``."""

    def __init__(self, dataset_param=None, model=None, *, files=None, dataset_dir: str = "", tokenizer=None,
                 spec: AnyResSpec = None, cutoff_len: int = 4096, image_loader=None, bos_id: int = None, eos_id: int = None):
        import os
        from .multimodal import ByteTokenizer, _read_records
        if dataset_param is not None:
            basic = dict(getattr(dataset_param, "basic_parameters", None) or {})
            files = files or basic.get("dataset") or basic.get("data_path")
            dataset_dir = basic.get("dataset_dir", dataset_dir)
            cutoff_len = int(basic.get("cutoff_len", cutoff_len))
        files = [files] if isinstance(files, str) else list(files)
        self.records = []
        for f in files:
            self.records += _read_records(f if os.path.isabs(f) or not dataset_dir else os.path.join(dataset_dir, f))
        self.dir, self.cutoff = dataset_dir, cutoff_len
        self.tok = tokenizer or ByteTokenizer()
        cfg = getattr(model, "config", None)
        if spec is None:
            vit = getattr(cfg, "vit", None)
            size = (vit.patch_size * vit.merge * 4) if vit is not None else 384
            spec = AnyResSpec(image_size=size, patch_size=vit.patch_size if vit else 16, downsample_ratio=vit.merge if vit else 2,
                              candidates=candidate_grid(size, 9), image_token_id=getattr(cfg, "image_token_id", 100003))
        self.spec, self.bos_id, self.eos_id = spec, bos_id, eos_id
        self.image_loader = image_loader or self._load

    def _load(self, p: str):
        import os
        from PIL import Image
        return Image.open(p if os.path.isabs(p) or not self.dir else os.path.join(self.dir, p))

    def _encode(self, s: str) -> List[int]:
        try:
            return list(self.tok.encode(s, add_special_tokens=False))      # transformers tokenizers
        except TypeError:
            return list(self.tok.encode(s))

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        from .multimodal import normalise_messages
        rec = self.records[i]
        msgs = [m for m in normalise_messages(rec) if m["role"] != "system"]
        turns = [(msgs[k]["content"], msgs[k + 1]["content"]) for k in range(0, len(msgs) - 1, 2)]
        paths = rec.get("images") or ([rec["image"]] if rec.get("image") else [])
        s = build_sft_sample(turns, [self.image_loader(p) for p in paths], self._encode, self.spec, self.bos_id, self.eos_id)
        if s["input_ids"].numel() > self.cutoff:          # cut text only after the last image placeholder
            last_img = int(s["images_seq_mask"].nonzero().max()) + 1 if s["images_seq_mask"].any() else 0
            keep = max(self.cutoff, last_img)
            for k in ("input_ids", "labels", "images_seq_mask"):
                s[k] = s[k][:keep]
        return s


def _register():
    from ..models.registry import data_register
    data_register.register("deepseekvl2")(TiledConversationDataset)


_register()


class TiledPackCollator:
    """Packs tiled samples into one token stream for the composable model: shifted labels, per-sample positions,
    ``cu_seqlens``, the ViT patch rows of every view and the tile grid of every image."""

    def __init__(self, patch: int, merge: int = 2, temporal: int = 1, ignore_id: int = -100):
        self.patch, self.merge, self.temporal, self.ignore = patch, merge, temporal, ignore_id

    def __call__(self, samples: Sequence[dict]) -> dict:
        ids, labels, pos, lens, views, crops = [], [], [], [], [], []
        for s in samples:
            n = s["input_ids"].numel()
            ids.append(s["input_ids"])
            lab = torch.full((n,), self.ignore, dtype=torch.long)
            lab[:-1] = s["labels"][1:]                                  # next-token targets inside the sample
            labels.append(lab)
            pos.append(torch.arange(n))
            lens.append(n)
            views.append(s["views"])
            crops.append(s["spatial_crop"])
        rows, grid = views_to_patch_rows(torch.cat(views), self.patch, self.merge, self.temporal)
        cu = torch.tensor([0] + lens, dtype=torch.int32).cumsum(0).to(torch.int32)
        return dict(input_ids=torch.cat(ids), labels=torch.cat(labels), position_ids=torch.cat(pos), cu_seqlens=cu,
                    max_seqlen=max(lens), pixel_values=rows, image_grid_thw=grid, spatial_crop=torch.cat(crops))
