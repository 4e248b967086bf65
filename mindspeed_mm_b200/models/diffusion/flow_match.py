"""Shifted flow-matching scheduler used by Wan (and, with other shifts, HunyuanVideo / FLUX).

Behaviour of ``WanFlowMatchScheduler`` (mindspeed_mm/models/diffusion/wan_flow_match_scheduler.py:8-160):
  sigma_i  = linspace(sigma_max, sigma_min, N [+1, last dropped when extra_one_step])
  sigma_i' = shift * sigma_i / (1 + (shift - 1) * sigma_i);   t_i = sigma_i' * num_train_timesteps
  x_t = (1 - sigma') x_0 + sigma' * noise;   target = noise - x_0
  loss = MSE(pred, target) * w(t),  w = a Gaussian bump around the middle timestep, shifted to min 0 and
  normalised to mean 1 over the table.  One timestep is drawn per micro-batch.  Sampling is Euler:
  x <- x + pred * (sigma_next - sigma), with optional classifier-free guidance.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..registry import model_register


@model_register.register("wan_flow_match_scheduler")
class FlowMatchScheduler:
    def __init__(self, num_inference_timesteps: Optional[int] = None, num_train_timesteps: int = 1000, shift: float = 3.0,
                 sigma_max: float = 1.0, sigma_min: float = 0.003 / 1.002, inverse_timesteps: bool = False,
                 extra_one_step: bool = False, reverse_sigmas: bool = False, guidance_scale: float = 0.0,
                 max_timestep_boundary: float = 1.0, min_timestep_boundary: float = 0.0, **_):
        if not (0 <= min_timestep_boundary < max_timestep_boundary <= 1):
            raise ValueError("min_timestep_boundary and max_timestep_boundary must satisfy 0 <= min < max <= 1")
        self.num_train_timesteps, self.shift = num_train_timesteps, shift
        self.sigma_max, self.sigma_min = sigma_max, sigma_min
        self.inverse_timesteps, self.extra_one_step, self.reverse_sigmas = inverse_timesteps, extra_one_step, reverse_sigmas
        self.guidance_scale = guidance_scale
        self.max_timestep_boundary, self.min_timestep_boundary = max_timestep_boundary, min_timestep_boundary
        self.num_inference_timesteps = num_inference_timesteps
        self.set_timesteps(num_inference_timesteps or num_train_timesteps, training=num_inference_timesteps is None)

    @property
    def do_classifier_free_guidance(self):
        return self.guidance_scale > 1.0

    def set_timesteps(self, num_steps: int, training: bool = False) -> None:
        n = num_steps + 1 if self.extra_one_step else num_steps
        s = torch.linspace(self.sigma_max, self.sigma_min, n)
        if self.extra_one_step:
            s = s[:-1]
        if self.inverse_timesteps:
            s = torch.flip(s, dims=[0])
        s = self.shift * s / (1 + (self.shift - 1) * s)
        if self.reverse_sigmas:
            s = 1 - s
        self.sigmas = s
        self.timesteps = s * self.num_train_timesteps
        if training:
            y = torch.exp(-2 * ((self.timesteps - num_steps / 2) / num_steps) ** 2)
            y = y - y.min()
            self.weights = y * (num_steps / y.sum())

    # ---- training ---------------------------------------------------------------------------
    def q_sample(self, latents, noise=None, t=None, generator=None, first_frame_latents=None):
        if noise is None:
            noise = torch.randn(latents.shape, generator=generator, device=latents.device, dtype=latents.dtype) \
                if generator is None or generator.device == latents.device else \
                torch.randn(latents.shape, generator=generator, dtype=latents.dtype).to(latents.device)
        if first_frame_latents is not None:
            noise[:, :, 0:1] = first_frame_latents
        if t is None:
            hi = int(self.max_timestep_boundary * self.num_train_timesteps)
            lo = int(self.min_timestep_boundary * self.num_train_timesteps)
            idx = torch.randint(lo, hi, (1,), generator=generator if generator is not None and generator.device.type == "cpu" else None)
        else:
            idx = torch.argmin((self.timesteps - t.detach().float().cpu().reshape(-1)[0]).abs()).reshape(1)
        sigma = self.sigmas[idx].to(latents.device, latents.dtype)
        timestep = self.timesteps[idx].to(latents.device)
        return (1 - sigma) * latents + sigma * noise, noise, timestep

    def training_weight(self, timestep) -> torch.Tensor:
        t = timestep.detach().float().cpu().reshape(-1)[0]
        return self.weights[torch.argmin((self.timesteps - t).abs())]

    def training_losses(self, model_output, x_start, noise, t, reduction: str = "mean", **_):
        target = noise - x_start
        loss = torch.nn.functional.mse_loss(model_output.float(), target.float(), reduction=reduction)
        return loss * self.training_weight(t).to(loss.device)

    # ---- sampling ---------------------------------------------------------------------------
    def step(self, model_output, timestep, sample):
        t = timestep.detach().float().cpu().reshape(-1)[0] if isinstance(timestep, torch.Tensor) else float(timestep)
        i = int(torch.argmin((self.timesteps - t).abs()))
        sigma = self.sigmas[i]
        nxt = (1.0 if (self.inverse_timesteps or self.reverse_sigmas) else 0.0) if i + 1 >= len(self.timesteps) \
            else self.sigmas[i + 1]
        return sample + model_output * (nxt - sigma)

    @torch.no_grad()
    def sample(self, model: Callable, latents, prompt_embeds, negative_prompt_embeds=None, progress: bool = False, **kw):
        it = self.timesteps
        if progress:
            from tqdm.auto import tqdm
            it = tqdm(it)
        for t in it:
            ts = t.expand(latents.shape[0]).to(latents.device)
            pred = model(latents, ts, prompt_embeds, **kw)
            if self.do_classifier_free_guidance and negative_prompt_embeds is not None:
                un = model(latents, ts, negative_prompt_embeds, **kw)
                pred = un + self.guidance_scale * (pred - un)
            latents = self.step(pred, t, latents)
        return latents
