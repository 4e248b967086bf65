"""Video / image transform pipelines built from a recipe's ``train_pipeline`` block.

``get_transforms(is_video, train_pipeline, image_size, transform_size)`` turns
``{"video": [{"trans_type": "ToTensorVideo"}, {"trans_type": "CenterCropResizeVideo", "param": {...}}, ...],
"image": [...]}`` into one callable, with the transform names and parameters of the reference's registry
(mindspeed_mm/data/data_utils/transform_pipeline.py:28-131, data_transform.py:283-1000) so data JSONs carry over.
Video clips are ``[T, C, H, W]`` tensors (uint8 from the reader, float in [0, 1] after ``ToTensorVideo``); image
pipelines take a PIL image or a ``[C, H, W]`` tensor.  All resampling is ``torch.nn.functional.interpolate``.
"""
from __future__ import annotations

import copy
import math
import random
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------ functional
def _check_clip(clip: torch.Tensor) -> None:
    if not torch.is_tensor(clip) or clip.dim() != 4:
        raise ValueError(f"a video clip is a 4-D tensor [T, C, H, W], got {type(clip).__name__} of dim {getattr(clip, 'dim', lambda: '?')()}")


def resize(clip, size: Sequence[int], mode: str = "bilinear", align_corners: bool = False, antialias: bool = False):
    kw = dict(align_corners=align_corners, antialias=antialias) if mode in ("bilinear", "bicubic") else {}
    return F.interpolate(clip, size=tuple(int(s) for s in size), mode=mode, **kw)


def crop(clip, top: int, left: int, h: int, w: int):
    return clip[..., top:top + h, left:left + w]


def center_crop(clip, size: Sequence[int]):
    h, w = clip.shape[-2:]
    th, tw = size
    if h < th or w < tw:
        raise ValueError(f"cannot centre-crop {h} x {w} to {th} x {tw}")
    return crop(clip, int(round((h - th) / 2.0)), int(round((w - tw) / 2.0)), th, tw)


def center_crop_short_edge(clip):
    h, w = clip.shape[-2:]
    s = min(h, w)
    return crop(clip, int(round((h - s) / 2.0)), int(round((w - s) / 2.0)), s, s)


def center_crop_to_ratio(clip, th: int, tw: int, top_crop: bool = False):
    """Largest centred (or top-anchored) crop with the aspect ratio th : tw."""
    h, w = clip.shape[-2:]
    r = th / tw
    nh, nw = (int(w * r), w) if h / w > r else (h, int(h / r))
    return crop(clip, 0 if top_crop else int(round((h - nh) / 2.0)), int(round((w - nw) / 2.0)), nh, nw)


def resize_crop_to_fill(clip, size: Sequence[int], mode: str = "bilinear"):
    """Scale so that the target is covered, then centre-crop to exactly ``size``."""
    h, w = clip.shape[-2:]
    th, tw = size
    rh, rw = th / h, tw / w
    if rh > rw:
        sh, sw = th, round(w * rh)
        clip = resize(clip, (sh, sw), mode)
        return crop(clip, 0, int(round(sw - tw) / 2.0), th, tw)
    sh, sw = round(h * rw), tw
    clip = resize(clip, (sh, sw), mode)
    return crop(clip, int(round(sh - th) / 2.0), 0, th, tw)


def long_side_size(h: int, w: int, size: Sequence[int], skip_low_resolution: bool = False) -> Tuple[int, int]:
    """Fit inside ``size`` keeping the aspect ratio (the longer side, relative to the box, reaches it)."""
    if h <= size[0] and w <= size[1] and skip_low_resolution:
        return h, w
    if h / w > size[0] / size[1]:
        return size[0], int(size[0] / h * w)
    return int(size[1] / w * h), size[1]


def short_side_size(h: int, w: int, size: Sequence[int], skip_low_resolution: bool = False) -> Tuple[int, int]:
    """Cover ``size`` keeping the aspect ratio."""
    if h <= size[0] and w <= size[1] and skip_low_resolution:
        return h, w
    if h / w < size[0] / size[1]:
        return size[0], int(size[0] / h * w)
    return int(size[1] / w * h), size[1]


def max_hw_size(h: int, w: int, max_hxw: int) -> Tuple[int, int]:
    if h * w > max_hxw:
        s = math.sqrt(max_hxw / (h * w))
        return int(h * s), int(w * s)
    return h, w


def _box(transform_size) -> Tuple[int, int]:
    if isinstance(transform_size, dict):
        return int(transform_size["max_height"]), int(transform_size["max_width"])
    if isinstance(transform_size, int):
        return transform_size, transform_size
    return tuple(int(s) for s in transform_size)


# ------------------------------------------------------------------------------------------ video transforms
class ToTensorVideo:
    """uint8 [T, C, H, W] (or [T, H, W, C]) -> float [T, C, H, W] in [0, 1]."""

    def __call__(self, clip):
        _check_clip(clip)
        if clip.shape[-1] in (1, 3) and clip.shape[1] not in (1, 3):
            clip = clip.permute(0, 3, 1, 2)
        return clip.float() / 255.0 if clip.dtype == torch.uint8 else clip.float()


class ToTensorAfterResize(ToTensorVideo):
    pass


class AENorm:
    """[0, 1] -> [-1, 1] (what the autoencoders were trained on)."""

    def __call__(self, clip):
        return 2.0 * clip - 1.0


class NormalizeVideo:
    def __init__(self, mean, std, inplace: bool = False):
        self.mean, self.std = torch.tensor(mean).view(-1, 1, 1), torch.tensor(std).view(-1, 1, 1)

    def __call__(self, clip):
        return (clip - self.mean.to(clip)) / self.std.to(clip)


class RandomHorizontalFlipVideo:
    def __init__(self, p: float = 0.5):
        self.p = p

    def __call__(self, clip):
        return clip.flip(-1) if random.random() < self.p else clip


class UCFCenterCropVideo:
    """Resize the short side to ``size`` and centre-crop the square (or ``size`` box)."""

    def __init__(self, size, interpolation_mode: str = "bilinear"):
        self.size, self.mode = _box(size), interpolation_mode

    def __call__(self, clip):
        _check_clip(clip)
        h, w = clip.shape[-2:]
        s = self.size[0] / min(h, w)
        clip = resize(clip, (max(self.size[0], round(h * s)), max(self.size[1], round(w * s))), self.mode)
        return center_crop(clip, self.size)


class CenterCropResizeVideo:
    """Centre crop to the target aspect ratio (or the short edge), then resize to the target box."""

    def __init__(self, transform_size="auto", use_short_edge: bool = False, top_crop: bool = False,
                 interpolation_mode: str = "bilinear", align_corners: bool = False, antialias: bool = False, size=None):
        self.size = _box(size if size is not None else transform_size)
        self.use_short_edge, self.top_crop = use_short_edge, top_crop
        self.mode, self.align_corners, self.antialias = interpolation_mode, align_corners, antialias

    def __call__(self, clip):
        _check_clip(clip)
        clip = center_crop_short_edge(clip) if self.use_short_edge else center_crop_to_ratio(clip, *self.size, self.top_crop)
        return resize(clip, self.size, self.mode, self.align_corners, self.antialias)


class CenterCropVideo:
    def __init__(self, size, interpolation_mode: str = "bilinear"):
        self.size = _box(size)

    def __call__(self, clip):
        return center_crop(clip, self.size)


class ResizeVideo:
    """``mode``: ``resize`` (to the box exactly), ``longside`` / ``shortside`` (aspect kept), ``hxw`` (cap on the area)."""

    def __init__(self, transform_size="auto", mode: str = "resize", interpolation_mode: str = "bilinear",
                 align_corners: bool = False, antialias: bool = False, skip_low_resolution: bool = False):
        self.how = mode
        self.area = int(transform_size["max_hxw"]) if (mode == "hxw" and isinstance(transform_size, dict)) else None
        self.size = _box(transform_size) if self.area is None and mode != "hxw" else None
        if mode == "hxw" and self.area is None:
            self.area = int(transform_size)
        self.mode, self.align_corners, self.antialias, self.skip = interpolation_mode, align_corners, antialias, skip_low_resolution

    def __call__(self, clip):
        _check_clip(clip)
        h, w = clip.shape[-2:]
        if self.how == "resize":
            th, tw = self.size
        elif self.how == "longside":
            th, tw = long_side_size(h, w, self.size, self.skip)
        elif self.how == "shortside":
            th, tw = short_side_size(h, w, self.size, self.skip)
        elif self.how == "hxw":
            th, tw = max_hw_size(h, w, self.area)
        else:
            raise NotImplementedError(f"ResizeVideo mode {self.how}")
        return clip if (th, tw) == (h, w) else resize(clip, (th, tw), self.mode, self.align_corners, self.antialias)


class LongSideResizeVideo(ResizeVideo):
    def __init__(self, size="auto", skip_low_resolution: bool = False, interpolation_mode: str = "bilinear",
                 align_corners: bool = False, antialias: bool = False, transform_size=None):
        super().__init__(transform_size if transform_size is not None else size, "longside", interpolation_mode,
                         align_corners, antialias, skip_low_resolution)


class MaxHWResizeVideo(ResizeVideo):
    def __init__(self, transform_size="auto", interpolation_mode: str = "bilinear", align_corners: bool = False,
                 antialias: bool = False):
        super().__init__(transform_size, "hxw", interpolation_mode, align_corners, antialias)


class SpatialStrideCropVideo:
    """Centred crop to multiples of ``stride`` (so that the autoencoder / patchifier divide the frame evenly)."""

    def __init__(self, stride: int):
        self.stride = stride

    def __call__(self, clip):
        h, w = clip.shape[-2:]
        ah, aw = h // self.stride * self.stride, w // self.stride * self.stride
        return crop(clip, (h - ah) // 2, (w - aw) // 2, ah, aw)


class ResizeCrop:
    """Resize (aspect kept) until the box is covered, then a random crop of the box."""

    def __init__(self, size, interpolation_mode: str = "bilinear"):
        self.size, self.mode = _box(size), interpolation_mode

    def __call__(self, clip):
        h, w = clip.shape[-2:]
        th, tw = self.size
        nh, nw = short_side_size(h, w, self.size)
        if (nh, nw) != (h, w):
            clip = resize(clip, (nh, nw), self.mode)
        top, left = random.randint(0, nh - th), random.randint(0, nw - tw)
        return crop(clip, top, left, th, tw)


class ResizeCropVideo(ResizeCrop):
    """Deterministic variant: centre crop after the covering resize."""

    def __call__(self, clip):
        return resize_crop_to_fill(clip, self.size, self.mode)


class ResizeCropToFill(ResizeCropVideo):
    pass


class ResizeToFill(ResizeCropVideo):
    pass


class RandomSizedCrop:
    """Random crop whose height and width are drawn from [size[0], size[1]], rounded down to multiples of 8."""

    def __init__(self, size):
        self.lo, self.hi = _box(size)

    def __call__(self, clip):
        H, W = clip.shape[-2:]
        h = min(H, random.randint(self.lo, self.hi)) // 8 * 8
        w = min(W, random.randint(self.lo, self.hi)) // 8 * 8
        return crop(clip, random.randint(0, H - h), random.randint(0, W - w), h, w)


class AffineVideo:
    """Small random rotation / translation / scale applied identically to every frame."""

    def __init__(self, degrees: float = 0.0, translate: float = 0.0, scale: Sequence[float] = (1.0, 1.0)):
        self.degrees, self.translate, self.scale = degrees, translate, tuple(scale)

    def __call__(self, clip):
        a = math.radians(random.uniform(-self.degrees, self.degrees))
        s = random.uniform(*self.scale)
        tx, ty = (random.uniform(-self.translate, self.translate) for _ in range(2))
        theta = torch.tensor([[math.cos(a) / s, -math.sin(a) / s, tx], [math.sin(a) / s, math.cos(a) / s, ty]], dtype=clip.dtype)
        grid = F.affine_grid(theta.expand(clip.shape[0], 2, 3), list(clip.shape), align_corners=False)
        return F.grid_sample(clip, grid, padding_mode="border", align_corners=False)


class TemporalRandomCrop:
    """``(begin, end)`` of a random window of ``size`` frames inside ``total_frames``."""

    def __init__(self, size: int):
        self.size = size

    def __call__(self, total_frames: int) -> Tuple[int, int]:
        begin = random.randint(0, max(0, total_frames - self.size - 1))
        return begin, min(begin + self.size, total_frames)


# ------------------------------------------------------------------------------------------ image transforms
def _to_chw(img) -> torch.Tensor:
    if torch.is_tensor(img):
        return img
    import numpy as np
    arr = torch.from_numpy(np.asarray(img.convert("RGB")).copy())
    return arr.permute(2, 0, 1)


class ToTensor:
    def __call__(self, img):
        t = _to_chw(img)
        return t.float() / 255.0 if t.dtype == torch.uint8 else t.float()


class _AsClip:
    """Runs a clip transform on one image ([C, H, W] <-> [1, C, H, W])."""

    def __init__(self, inner):
        self.inner = inner

    def __call__(self, img):
        t = _to_chw(img)
        was_u8 = t.dtype == torch.uint8
        out = self.inner(t.float().unsqueeze(0)).squeeze(0)
        return out.round().clamp(0, 255).to(torch.uint8) if was_u8 else out


class CenterCropArr:
    """Centre crop of a square of side ``size`` after scaling the short side to it (ADM-style)."""

    def __init__(self, size: int = 256):
        self.inner = UCFCenterCropVideo(size, "bicubic")

    def __call__(self, img):
        return _AsClip(self.inner)(img)


class Expand2Square:
    """Pad to a square with the mean colour (LLaVA-style), image centred."""

    def __init__(self, mean: Sequence[float] = (0.48145466, 0.4578275, 0.40821073)):
        self.mean = mean

    def __call__(self, img):
        t = _to_chw(img)
        c, h, w = t.shape
        s = max(h, w)
        fill = torch.tensor(self.mean).view(-1, 1, 1) * (255.0 if t.dtype == torch.uint8 else 1.0)
        out = fill.to(t.dtype).expand(c, s, s).clone()
        top, left = (s - h) // 2, (s - w) // 2
        out[:, top:top + h, left:left + w] = t
        return out


class Resize:
    def __init__(self, size, interpolation: str = "BILINEAR", antialias: bool = True):
        self.size = _box(size)
        self.mode = {"BICUBIC": "bicubic", "BILINEAR": "bilinear", "NEAREST": "nearest", "NEAREST_EXACT": "nearest-exact",
                     "BOX": "area", "HAMMING": "bilinear", "LANCZOS": "bicubic"}[str(interpolation).upper()]
        self.antialias = antialias

    def __call__(self, img):
        return _AsClip(lambda c: resize(c, self.size, self.mode, antialias=self.antialias and self.mode in ("bilinear", "bicubic")))(img)


class RandomHorizontalFlip(RandomHorizontalFlipVideo):
    def __call__(self, img):
        t = _to_chw(img)
        return t.flip(-1) if random.random() < self.p else t


class Lambda:
    def __init__(self, lambd: Callable):
        self.fn = lambd

    def __call__(self, x):
        return self.fn(x)


VIDEO_TRANSFORMS: Dict[str, type] = {
    "ToTensorVideo": ToTensorVideo, "ToTensorAfterResize": ToTensorAfterResize, "RandomHorizontalFlipVideo": RandomHorizontalFlipVideo,
    "UCFCenterCropVideo": UCFCenterCropVideo, "ResizeCrop": ResizeCrop, "RandSizeCropArr": RandomSizedCrop,
    "RandomSizedCrop": RandomSizedCrop, "CenterCropResizeVideo": CenterCropResizeVideo, "LongSideResizeVideo": LongSideResizeVideo,
    "ResizeVideo": ResizeVideo, "SpatialStrideCropVideo": SpatialStrideCropVideo, "norm_fun": NormalizeVideo, "ae_norm": AENorm,
    "MaxHWResizeVideo": MaxHWResizeVideo, "Resize": lambda **kw: _ClipResize(**kw), "CenterCropVideo": CenterCropVideo,
    "AffineVideo": AffineVideo, "ResizeCropVideo": ResizeCropVideo, "ResizeToFill": ResizeToFill,
}
IMAGE_TRANSFORMS: Dict[str, type] = {
    "Lambda": Lambda, "ToTensorVideo": lambda **kw: _AsClip(ToTensorVideo(**kw)),
    "CenterCropResizeVideo": lambda **kw: _AsClip(CenterCropResizeVideo(**kw)), "CenterCropArr": CenterCropArr,
    "ResizeCropToFill": lambda **kw: _AsClip(ResizeCropToFill(**kw)), "RandomHorizontalFlip": RandomHorizontalFlip,
    "ToTensor": ToTensor, "norm_fun": NormalizeVideo, "ae_norm": AENorm, "Pad2Square": Expand2Square, "Resize": Resize,
    "ResizeToFill": lambda **kw: _AsClip(ResizeToFill(**kw)),
}


class _ClipResize:
    def __init__(self, size, interpolation: str = "BILINEAR", antialias: bool = True):
        self.inner = Resize(size, interpolation, antialias)

    def __call__(self, clip):
        return resize(clip, self.inner.size, self.inner.mode, antialias=self.inner.antialias and self.inner.mode in ("bilinear", "bicubic"))


class Compose:
    def __init__(self, steps: List[Callable]):
        self.steps = steps

    def __call__(self, x):
        for s in self.steps:
            x = s(x)
        return x


def get_transforms(is_video: bool = True, train_pipeline: Optional[dict] = None, image_size=None, transform_size=None):
    """Build the pipeline of one modality.  ``"size": "auto"`` / ``"transform_size": "auto"`` parameters take the values the
    dataset passes (per-sample buckets of dynamic-resolution datasets)."""
    if train_pipeline is None:
        return None
    table = VIDEO_TRANSFORMS if is_video else IMAGE_TRANSFORMS
    steps = []
    for entry in copy.deepcopy(train_pipeline.get("video" if is_video else "image", [])):
        param = dict(entry.get("param") or {})
        if image_size and param.get("size") == "auto":
            param["size"] = image_size
        elif transform_size and param.get("transform_size") == "auto":
            param["transform_size"] = transform_size
        name = entry.get("trans_type", "")
        if name not in table:
            raise NotImplementedError(f"unsupported {'video' if is_video else 'image'} transform type: {name}")
        steps.append(table[name](**param))
    return Compose(steps)
