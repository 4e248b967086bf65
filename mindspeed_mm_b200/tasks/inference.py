"""Inference pipelines.

* ``VLMGenerator``      - greedy / top-p decoding for the packed Qwen2.5-VL model with a growing sequence (the
                          training kernels are prefill-shaped; every step re-runs the packed forward on the
                          prefix, which is exact and adequate for evaluation-sized generations).
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
        c, v = model.config, model.config.vision
        self.collator = PackedVLMCollator(c.image_token_id, c.vision_start_token_id, v.spatial_merge_size, v.patch_size,
                                          v.window_size, v.hidden_size // v.num_heads)

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
    def generate(self, input_ids, pixel_values=None, image_grid_thw=None, max_new_tokens: int = 16, temperature: float = 0.0,
                 top_p: float = 1.0, device="cpu", generator=None) -> torch.Tensor:
        ids = input_ids.clone()
        for _ in range(max_new_tokens):
            logits = self.next_logits(ids, pixel_values, image_grid_thw, device)
            if temperature <= 0:
                nxt = int(logits.argmax())
            else:
                p = torch.softmax(logits / temperature, -1)
                sp, si = torch.sort(p, descending=True)
                keep = (sp.cumsum(0) - sp) < top_p
                sp = sp * keep
                nxt = int(si[torch.multinomial(sp / sp.sum(), 1, generator=generator)])
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
