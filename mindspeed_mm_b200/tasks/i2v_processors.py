"""Image-to-video conditioning builders: what each model family feeds its DiT besides the noisy latents.

A processor is ``proc(vae, videos [B, C, T, H, W] in [-1, 1], video_latents [B, c, t, h, w], **extras) -> dict`` of extra
batch entries; ``build_i2v_processor(config)`` picks one by ``processor_id`` (reference:
mindspeed_mm/utils/extra_processor/i2v_processors.py:1-35, called from mindspeed_mm/models/ae/base.py:50-54).

* ``cogvideox``  -- first frame + log-normal noise (sigma = exp(N(-3, 0.5))) -> VAE -> zero-padded (or repeated) over time,
  dropped to zeros with probability ``noised_image_dropout`` (cogvideox_i2v_processor.py:5-56).
* ``stepvideo``  -- same noise, latent padded with zeros over time (stepvideo_i2v_processor.py:4-31).
* ``opensoraplan`` -- VAE latents of the masked video + the pixel mask folded to latent resolution: every ``stride_t``
  frames (the first frame alone) and every ``stride_h x stride_w`` pixel block become channels (opensoraplan_i2v_processor.py).
* ``hunyuanvideo`` -- first-frame latents decoded and re-encoded as the condition latent, plus the decoded picture for the
  semantic (vision-language) branch, blacked out with probability ``sematic_cond_drop_p`` (hunyuanvideo_i2v_processor.py).
* ``hunyuanvideo_15`` -- condition tensor with one extra mask channel: first-frame latents in frame 0, mask = 1 there; the
  first frame is also passed through a vision tower (SigLIP in the released model) (hunyuanvideo_15_i2v_processor.py:223-278).
* ``wan`` / ``wan_ti2v`` -- live in ``tasks/inference.py: wan_i2v_condition`` and ``models/wan_variants.py: ti2v_timesteps``.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F


def _randn_like(x: torch.Tensor, g: Optional[torch.Generator]) -> torch.Tensor:
    return torch.randn(x.shape, generator=g, dtype=torch.float32).to(x.device, x.dtype)


def add_lognormal_noise(image: torch.Tensor, g: Optional[torch.Generator] = None, mean: float = -3.0, std: float = 0.5):
    """image [B, ...]: one noise level per sample, sigma = exp(N(mean, std))."""
    sigma = torch.exp(torch.randn(image.shape[0], generator=g) * std + mean).to(image.device, image.dtype)
    return image + _randn_like(image, g) * sigma.view(-1, *([1] * (image.dim() - 1)))


class _Seeded:
    def __init__(self, seed: int = 0):
        self.generator = torch.Generator().manual_seed(seed)

    def _coin(self, p: float) -> bool:
        return p > 0 and float(torch.rand((), generator=self.generator)) < p


class CogVideoXI2V(_Seeded):
    def __init__(self, config: dict = None, seed: int = 0):
        super().__init__(seed)
        c = config or {}
        self.all_concat = bool(c.get("noised_image_all_concat", False))
        self.dropout = float(c.get("noised_image_dropout", 0.05))
        self.noised = bool(c.get("noised_image_input", True))

    def __call__(self, vae, videos, video_latents, images=None, **_):
        if self._coin(self.dropout):
            return {"masked_video": torch.zeros_like(video_latents)}
        img = (videos[:, :, :1] if images is None else images).to(videos.dtype)
        if self.noised:
            img = add_lognormal_noise(img, self.generator)
        lat = vae.encode(img).to(video_latents.dtype)
        t = video_latents.shape[2]
        if self.all_concat:
            lat = lat.repeat(1, 1, t, 1, 1)
        else:
            lat = torch.cat([lat, torch.zeros_like(video_latents[:, :, 1:])], 2)
        return {"masked_video": lat}


class StepVideoI2V(_Seeded):
    def __call__(self, vae, videos, video_latents, images=None, **_):
        img = (videos[:, :, :1] if images is None else images).to(videos.dtype)
        lat = vae.encode(add_lognormal_noise(img, self.generator)).to(video_latents.dtype)
        return {"image_latents": torch.cat([lat, torch.zeros_like(video_latents[:, :, 1:])], 2)}


def compress_mask(mask: torch.Tensor, stride_t: int = 4, stride_h: int = 8, stride_w: int = 8) -> torch.Tensor:
    """mask [B, 1, T, H, W] with T = 1 + k * stride_t -> [B, stride_t * stride_h * stride_w, 1 + k, H / sh, W / sw]: the
    first frame is repeated ``stride_t`` times so that it fills a temporal group of its own, then time groups and pixel
    blocks are moved into channels."""
    B, _, T, H, W = mask.shape
    m = torch.cat([mask[:, :, :1].repeat(1, 1, stride_t, 1, 1), mask[:, :, 1:]], 2)
    t = m.shape[2] // stride_t
    m = m.view(B, t, stride_t, H // stride_h, stride_h, W // stride_w, stride_w)
    return m.permute(0, 2, 4, 6, 1, 3, 5).reshape(B, stride_t * stride_h * stride_w, t, H // stride_h, W // stride_w)


class OpenSoraPlanI2V:
    def __init__(self, config: dict = None, seed: int = 0):
        c = config or {}
        self.strides = (int(c.get("ae_stride_t", 4)), int(c.get("ae_stride_h", 8)), int(c.get("ae_stride_w", 8)))

    def __call__(self, vae, videos, video_latents, masked_video=None, input_mask=None, **_):
        if masked_video is None or input_mask is None:
            raise ValueError("the Open-Sora-Plan processor needs 'masked_video' and 'input_mask' in the batch")
        return {"masked_video": vae.encode(masked_video.to(videos.dtype)).to(video_latents.dtype),
                "input_mask": compress_mask(input_mask.to(videos.dtype), *self.strides)}


class HunyuanVideoI2V(_Seeded):
    """``image_preprocess(images [B, 3, H, W] in [0, 1]) -> tensor`` prepares the picture for the semantic branch (CLIP-style
    resize + normalise by default)."""

    def __init__(self, config: dict = None, seed: int = 0, image_preprocess: Optional[Callable] = None):
        super().__init__(seed)
        c = config or {}
        self.drop = float(c.get("sematic_cond_drop_p", 0.0))
        self.size = int(c.get("image_size", 336))
        self.pre = image_preprocess or self._clip_like

    def _clip_like(self, img):
        from ..data.synthetic import CLIP_MEAN, CLIP_STD
        img = F.interpolate(img.float(), size=(self.size, self.size), mode="bicubic", align_corners=False, antialias=True).clamp(0, 1)
        mean = torch.tensor(CLIP_MEAN, device=img.device).view(1, 3, 1, 1)
        std = torch.tensor(CLIP_STD, device=img.device).view(1, 3, 1, 1)
        return (img - mean) / std

    def __call__(self, vae, videos, video_latents, **_):
        scale = float(getattr(vae, "scaling_factor", 1.0))
        first = video_latents[:, :, :1] / scale
        pictures = (vae.decode(first)[:, :, 0] / 2 + 0.5).clamp(0, 1)                       # [B, 3, H, W] in [0, 1]
        pictures = (pictures * 255).round() / 255                                           # 8-bit round trip of the reference
        cond = vae.encode(((pictures - 0.5) / 0.5).unsqueeze(2).to(video_latents.dtype))
        uncond = self._coin(self.drop)
        semantic = torch.zeros_like(pictures) if uncond else pictures
        return {"cond_latents": cond.to(video_latents.dtype), "pixel_value_llava": self.pre(semantic),
                "uncond": torch.tensor(int(uncond))}


class HunyuanVideo15I2V:
    """``vision_tower(images uint8-range [B, 3, H, W] in [0, 1]) -> [B, L, D]`` is optional; without it only the condition
    latents are produced."""

    def __init__(self, config: dict = None, seed: int = 0, vision_tower: Optional[Callable] = None):
        self.vision_tower = vision_tower

    def __call__(self, vae, videos, video_latents, **_):
        b, c, f, h, w = video_latents.shape
        cond = video_latents.new_zeros(b, c + 1, f, h, w)
        cond[:, :c, :1] = video_latents[:, :, :1]
        cond[:, c, 0] = 1
        out = {"cond_latents": cond}
        if self.vision_tower is not None:
            first = videos[:, :, 0]
            if float(first.max()) > 1.0 or float(first.min()) < -1.0:
                raise ValueError("frames must be in [-1, 1]")
            with torch.no_grad():
                out["vision_states"] = self.vision_tower(((first + 1) / 2 * 255).round().clamp(0, 255) / 255)
        return out


class WanI2V:
    """Thin adapter so that the Wan builder is reachable through the same factory."""

    def __init__(self, config: dict = None, seed: int = 0, clip_vision=None):
        self.clip = clip_vision

    def __call__(self, vae, videos, video_latents, **_):
        from .inference import wan_i2v_condition
        res = wan_i2v_condition(videos[:, :, 0], vae, self.clip, frames=videos.shape[2])
        return res if isinstance(res, dict) else {"first_frame_latents": res[0], "clip_feature": res[1]}


PROCESSORS: Dict[str, type] = {"cogvideox_i2v_processor": CogVideoXI2V, "stepvideo_i2v_processor": StepVideoI2V,
                               "opensoraplan_i2v_processor": OpenSoraPlanI2V, "hunyuanvideo_i2v_processor": HunyuanVideoI2V,
                               "hunyuanvideo_15_i2v_processor": HunyuanVideo15I2V, "wan_i2v_processor": WanI2V}


def build_i2v_processor(config: Optional[dict], **kw):
    if not config:
        return None
    pid = config.get("processor_id") or config.get("model_id")
    if pid not in PROCESSORS:
        raise ValueError(f"unknown i2v processor {pid!r}; known: {sorted(PROCESSORS)}")
    return PROCESSORS[pid](config, **kw)
