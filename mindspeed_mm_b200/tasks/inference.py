"""Inference pipelines.

* ``VLMGenerator``      - greedy / top-p decoding for the packed Qwen2.5-VL / Qwen3-VL models with a per-layer key / value cache:
                          the prompt (vision tower included) runs once, every later step feeds one token whose
                          attention reads the cached keys and values (``use_cache=False`` re-runs the whole prefix
                          per token instead, the exact but quadratic form).
* ``WanPipeline``       - text-to-video / image-to-video sampling: flow-matching Euler steps with classifier-free
                          guidance over the DiT, latents decoded by an optional VAE callable.
Reference: mindspeed_mm/tasks/inference/pipeline/{qwen2vl_pipeline.py, wan_pipeline.py} and the generation mixin;
mindspeed_mm/fsdp/inference/inference_runner.py:37.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..data.collate import PackedVLMCollator
from ..models.diffusion import FlowMatchScheduler


class VLMGenerator:
    def __init__(self, model, run: Optional[Callable] = None, eos_token_id: Optional[int] = None):
        self.model, self.run, self.eos = model, run, eos_token_id
        self.collator = PackedVLMCollator.for_config(model.config)

    @torch.no_grad()
    def next_logits(self, input_ids, pixel_values=None, image_grid_thw=None, device="cpu"):
        sample = dict(input_ids=input_ids, labels=input_ids.clone())
        if pixel_values is not None:
            sample.update(pixel_values=pixel_values, image_grid_thw=image_grid_thw)
        b = self.collator([sample])
        b.pop("labels")
        b = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in b.items()}
        if "vision_plan" in b:
            b["vision_plan"] = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in b["vision_plan"].items()}
        logits = self.model(b, run=self.run)
        return logits[-1].float()

    @torch.no_grad()
    def _prefill(self, input_ids, pixel_values, image_grid_thw, device):
        sample = dict(input_ids=input_ids, labels=input_ids.clone())
        if pixel_values is not None:
            sample.update(pixel_values=pixel_values, image_grid_thw=image_grid_thw)
        b = self.collator([sample])
        b.pop("labels")
        next_pos = int(b["position_ids"].max()) + 1          # where the text continues on all three rotary axes
        b = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in b.items()}
        if "vision_plan" in b:
            b["vision_plan"] = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in b["vision_plan"].items()}
        cache = [dict() for _ in self.model.layers]
        logits = self.model(b, run=self.run, kv_cache=cache)
        return logits[-1].float(), cache, next_pos

    @torch.no_grad()
    def _decode(self, token: int, pos: int, cache, device):
        b = dict(input_ids=torch.tensor([token], device=device),
                 position_ids=torch.full((3, 1), pos, dtype=torch.long, device=device))
        return self.model(b, run=self.run, kv_cache=cache)[-1].float()

    @staticmethod
    def _pick(logits, temperature, top_p, generator):
        if temperature <= 0:
            return int(logits.argmax())
        p = torch.softmax(logits / temperature, -1)
        sp, si = torch.sort(p, descending=True)
        keep = (sp.cumsum(0) - sp) < top_p
        sp = sp * keep
        return int(si[torch.multinomial(sp / sp.sum(), 1, generator=generator)])

    @torch.no_grad()
    def generate(self, input_ids, pixel_values=None, image_grid_thw=None, max_new_tokens: int = 16, temperature: float = 0.0,
                 top_p: float = 1.0, device="cpu", generator=None, use_cache: bool = True) -> torch.Tensor:
        ids = input_ids.clone()
        cache, pos = None, 0
        for step in range(max_new_tokens):
            if not use_cache:
                logits = self.next_logits(ids, pixel_values, image_grid_thw, device)
            elif cache is None:
                logits, cache, pos = self._prefill(ids, pixel_values, image_grid_thw, device)
            else:
                logits = self._decode(int(ids[-1]), pos, cache, device)
                pos += 1
            nxt = self._pick(logits.cpu(), temperature, top_p, generator)
            ids = torch.cat([ids, torch.tensor([nxt])])
            if self.eos is not None and nxt == self.eos:
                break
        return ids


class WanPipeline:
    def __init__(self, dit, scheduler: Optional[FlowMatchScheduler] = None, vae_decode: Optional[Callable] = None,
                 text_encode: Optional[Callable] = None, run: Optional[Callable] = None):
        self.dit, self.vae_decode, self.text_encode, self.run = dit, vae_decode, text_encode, run
        self.scheduler = scheduler or FlowMatchScheduler(num_inference_timesteps=50, shift=5.0, sigma_min=0.0,
                                                         extra_one_step=True, guidance_scale=5.0)

    @torch.no_grad()
    def __call__(self, prompt_embeds, negative_prompt_embeds=None, frames: int = 21, height: int = 60, width: int = 104,
                 generator=None, clip_feature=None, device="cpu", dtype=torch.float32):
        if self.text_encode is not None and not isinstance(prompt_embeds, torch.Tensor):
            prompt_embeds = self.text_encode(prompt_embeds)
        B = prompt_embeds.shape[0]
        c = self.dit.config
        lat = torch.randn(B, c.in_dim, frames, height, width, generator=generator, dtype=torch.float32).to(device, dtype)
        fn = lambda x, t, p: self.dit(x, t, p, clip_feature, run=self.run)      # noqa: E731
        lat = self.scheduler.sample(fn, lat, prompt_embeds.to(device, dtype),
                                    None if negative_prompt_embeds is None else negative_prompt_embeds.to(device, dtype))
        return self.vae_decode(lat) if self.vae_decode is not None else lat


def wan_i2v_condition(first_frame, vae, clip_vision=None, frames: int = 81, last_frame=None):
    """Image-to-video conditioning of Wan (mindspeed_mm/utils/extra_processor/wan_i2v_processor.py): the first
    (and optionally last) frame padded with zeros to ``frames`` is VAE-encoded, a 4-channel mask marks which latent
    frames are given (the first pixel frame repeated 4x so that it folds onto one latent frame), and the CLIP
    penultimate-layer tokens of the image feed the DiT's image cross-attention.

    first_frame: [B, 3, H, W] in [-1, 1].  Returns ``(y [B, 4 + z, 1 + (frames-1)/4, H/8, W/8], clip_feature)``."""
    B, _, H, W = first_frame.shape
    video = torch.zeros(B, 3, frames, H, W, dtype=first_frame.dtype, device=first_frame.device)
    video[:, :, 0] = first_frame
    mask = torch.zeros(B, frames, H // 8, W // 8, dtype=first_frame.dtype, device=first_frame.device)
    mask[:, 0] = 1
    if last_frame is not None:
        video[:, :, -1] = last_frame
        mask[:, -1] = 1
    lat = vae.encode(video)
    mask = torch.cat([mask[:, :1].repeat(1, 4, 1, 1), mask[:, 1:]], dim=1)          # 4 + (frames - 1)
    mask = mask.view(B, mask.shape[1] // 4, 4, H // 8, W // 8).transpose(1, 2)      # [B, 4, T_lat, h, w]
    clip = None
    if clip_vision is not None:
        img = torch.nn.functional.interpolate(first_frame.float(), size=(clip_vision.c.image_size,) * 2, mode="bicubic",
                                              align_corners=False)
        mean = torch.tensor([0.48145466, 0.4578275, 0.40821073], device=img.device).view(1, 3, 1, 1)
        std = torch.tensor([0.26862954, 0.26130258, 0.27577711], device=img.device).view(1, 3, 1, 1)
        clip = clip_vision.encode(((img * 0.5 + 0.5) - mean) / std)
    return torch.cat([mask, lat], dim=1), clip


class MMDiTPipeline:
    """Text-to-image / text-to-video sampling for the dual/single-stream DiTs (FLUX, SD3, HunyuanVideo):
    flow-matching Euler steps with an optional distilled-guidance input and classifier-free guidance
    (mindspeed_mm/tasks/inference/pipeline/hunyuanvideo_pipeline.py, flux pipelines of the diffusers examples)."""

    def __init__(self, dit, scheduler: Optional[FlowMatchScheduler] = None, vae_decode: Optional[Callable] = None,
                 run: Optional[Callable] = None, embedded_guidance: Optional[float] = None):
        self.dit, self.vae_decode, self.run, self.embedded_guidance = dit, vae_decode, run, embedded_guidance
        self.scheduler = scheduler or FlowMatchScheduler(num_inference_timesteps=28, shift=3.0, sigma_min=0.0,
                                                         extra_one_step=True, guidance_scale=1.0)

    @torch.no_grad()
    def __call__(self, txt, pooled, negative=None, frames: int = 1, height: int = 64, width: int = 64, generator=None,
                 device="cpu", dtype=torch.float32):
        c = self.dit.config
        B = txt.shape[0]
        lat = torch.randn(B, c.in_channels, frames, height, width, generator=generator, dtype=torch.float32).to(device, dtype)
        g = None if self.embedded_guidance is None else torch.full((B,), self.embedded_guidance, device=device, dtype=dtype)

        def fn(x, t, cond):
            te, po = cond
            return self.dit(x, t, te, po, g, run=self.run)
        neg = None if negative is None else (negative[0].to(device, dtype), negative[1].to(device, dtype))
        lat = self.scheduler.sample(fn, lat, (txt.to(device, dtype), pooled.to(device, dtype)), neg)
        return self.vae_decode(lat) if self.vae_decode is not None else lat


class TextToVideoPipeline:
    """Sampling loop shared by the cross-attention and joint-sequence video DiTs (``models/video_dits.py``) with any scheduler
    of ``models/diffusion``: CogVideoX (zero-SNR v-prediction + dynamic guidance), Open-Sora-Plan (linear-quadratic flow
    schedule), StepVideo and HunyuanVideo style discrete flow matching, Open-Sora rectified flow, DDPM / DDIM
    (mindspeed_mm/tasks/inference/pipeline/{cogvideox,opensoraplan,stepvideo,hunyuanvideo}_pipeline.py).

    ``dit(latents, t, text, text_mask)`` is the denoiser; schedulers receive it wrapped as ``model(x, t, **kwargs)`` with
    the positive prompt in ``model_kwargs`` and the negative prompt in ``negative_kwargs``."""

    PRESETS = {
        "cogvideox": dict(model_id="cogvideo_diffusion", num_inference_steps=50, guidance_scale=6.0),
        "opensoraplan": dict(model_id="opensoraplan_v1_5", num_inference_steps=50, guidance_scale=4.5),
        "stepvideo": dict(model_id="flow_match_discrete", num_inference_timesteps=50, shift=13.0, guidance_scale=9.0),
        "hunyuanvideo": dict(model_id="flow_match_discrete", num_inference_timesteps=50, shift=7.0, guidance_scale=1.0,
                             embedded_guidance_scale=6.0),
        "opensora": dict(model_id="rflow", num_inference_steps=30, cfg_scale=7.0),
    }

    def __init__(self, dit, scheduler=None, vae_decode: Optional[Callable] = None, text_encode: Optional[Callable] = None,
                 run: Optional[Callable] = None, preset: Optional[str] = None):
        from ..models.diffusion import build_scheduler
        self.dit, self.vae_decode, self.text_encode, self.run = dit, vae_decode, text_encode, run
        self.scheduler = scheduler if scheduler is not None else build_scheduler(self.PRESETS[preset or "stepvideo"])

    def _model(self, x, t, text=None, text_mask=None, **extra):
        if text.shape[0] != x.shape[0]:
            text = text.expand(x.shape[0], -1, -1) if text.shape[0] == 1 else text.repeat(x.shape[0] // text.shape[0], 1, 1)
            if text_mask is not None:
                text_mask = text_mask.expand(x.shape[0], -1) if text_mask.shape[0] == 1 else text_mask.repeat(x.shape[0] // text_mask.shape[0], 1)
        kw = {"run": self.run} if self.run is not None else {}
        return self.dit(x, t.reshape(-1).expand(x.shape[0]) if t.numel() == 1 else t, text, text_mask, **kw)

    @torch.no_grad()
    def __call__(self, prompt_embeds, negative_prompt_embeds=None, prompt_mask=None, negative_mask=None, frames: int = 13,
                 height: int = 32, width: int = 32, generator=None, device="cpu", dtype=torch.float32, **sample_kw):
        if self.text_encode is not None and not isinstance(prompt_embeds, torch.Tensor):
            prompt_embeds = self.text_encode(prompt_embeds)
        B = prompt_embeds.shape[0]
        C = self.dit.config.in_channels
        lat = torch.randn(B, C, frames, height, width, generator=generator, dtype=torch.float32).to(device, dtype)
        pos = dict(text=prompt_embeds.to(device, dtype), text_mask=prompt_mask)
        neg = None if negative_prompt_embeds is None else dict(text=negative_prompt_embeds.to(device, dtype), text_mask=negative_mask)
        sched = self.scheduler
        if type(sched).__name__ in ("RFlow", "GaussianDiffusion", "DDPM", "IDDPM"):
            # these samplers run cond / uncond as one doubled batch
            text = pos["text"] if neg is None else torch.cat([pos["text"], neg["text"]])
            mask = None
            if prompt_mask is not None:
                mask = prompt_mask if neg is None else torch.cat([prompt_mask, negative_mask if negative_mask is not None else prompt_mask])
            guided = neg is not None
            if not guided:
                sample_kw.setdefault("guidance_scale", 1.0)
            fn = (lambda x, t, **kw: self._model(x, t, text=text if x.shape[0] == text.shape[0] else pos["text"],
                                                 text_mask=mask if mask is None or x.shape[0] == mask.shape[0] else prompt_mask))
            if type(sched).__name__ == "RFlow" and not guided:
                fn = (lambda x, t, **kw: self._model(x, t, text=torch.cat([pos["text"], pos["text"]]), text_mask=None if prompt_mask is None
                                                     else torch.cat([prompt_mask, prompt_mask])))
            lat = sched.sample(fn, lat, model_kwargs={}, **sample_kw)
        else:
            lat = sched.sample(self._model, lat, model_kwargs=pos, negative_kwargs=neg, **sample_kw)
        return self.vae_decode(lat) if self.vae_decode is not None else lat
