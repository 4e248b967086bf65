"""Flow-matching and v-prediction schedulers of the generation model zoo other than Wan's.

* ``RFlow``                      -- rectified flow of Open-Sora (mindspeed_mm/models/diffusion/rflow.py:35): x_t = (1 - s) x0 +
  s * noise with s = t / T, logit-normal or uniform t, resolution / length dependent timestep transform, Euler sampler
  with classifier-free guidance and optional frame mask.
* ``FlowMatchDiscreteScheduler`` -- HunyuanVideo (flow_match_discrete_scheduler.py:29): sigmas on a shifted grid
  ``shift * s / (1 + (shift - 1) s)``, density-sampled training indices, Euler steps, optional preconditioned outputs.
* ``HunyuanVideo15Scheduler``    -- HunyuanVideo-1.5 (hunyuan_video_15_scheduler.py:135): same solver, timestep sampler with
  uniform / logit-normal SNR types and a train-time shift.
* ``OpenSoraPlanScheduler``      -- Open-Sora-Plan v1.5 (opensoraplanv1_5_scheduler.py:62): sigma density sampling
  (logit-normal / mode / uniform), SD3 loss weighting (sigma_sqrt / cosmap), linear-quadratic inference grid.
* ``CogVideoDiffusion``          -- CogVideoX (cogvideo_diffusion.py:249): zero-terminal-SNR DDPM discretisation, v-prediction
  through ``c_skip / c_out`` scaling, 1 / (1 - alpha) loss weight with optional min-SNR cap, DDIM-style sampler with the
  dynamic guidance ramp.

All of them share ``q_sample -> (x_t, noise, t)``, ``training_losses(model_output, x_start, noise=..., t=...) -> [B]`` and
``sample(model, latents, ...)`` so the SoRA model can swap them by ``model_id``.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from .gaussian import mean_flat, randn_like


def _bcast(v: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return v.to(like.device, torch.float32).reshape(-1, *([1] * (like.dim() - 1)))


def density_sample(scheme: str, n: int, logit_mean: float = 0.0, logit_std: float = 1.0, mode_scale: float = 1.29,
                   generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """u in (0, 1) for timestep / sigma selection (the SD3 weighting schemes)."""
    if scheme in ("logit_normal", "logit-normal"):
        return torch.sigmoid(torch.randn(n, generator=generator) * logit_std + logit_mean)
    u = torch.rand(n, generator=generator)
    if scheme == "mode":
        return 1 - u - mode_scale * (torch.cos(math.pi * u / 2) ** 2 - 1 + u)
    return u


def rescale_noise_cfg(noise_cfg, noise_pred_text, guidance_rescale: float = 0.0):
    """Pulls the guided prediction's per-sample std back toward the conditional one (fixes over-exposure)."""
    if guidance_rescale <= 0:
        return noise_cfg
    dims = list(range(1, noise_pred_text.dim()))
    rescaled = noise_cfg * (noise_pred_text.std(dim=dims, keepdim=True) / noise_cfg.std(dim=dims, keepdim=True))
    return guidance_rescale * rescaled + (1 - guidance_rescale) * noise_cfg


# ------------------------------------------------------------------------------------------------- RFlow
def resolution_timestep_transform(t, height, width, num_frames, base_resolution=512 * 512, base_num_frames=1, scale=1.0,
                                  num_timesteps=1):
    """Larger / longer videos are pushed toward noisier timesteps: t' = r t / (1 + (r - 1) t), r = sqrt(area ratio) *
    sqrt(latent-frame ratio) (rflow.py:9; 17 pixel frames = 5 latent frames)."""
    t = t / num_timesteps
    ratio_space = (height.float() * width.float() / base_resolution).sqrt()
    frames = torch.where(num_frames == 1, torch.ones_like(num_frames), num_frames // 17 * 5).float()
    ratio = ratio_space * (frames / base_num_frames).sqrt() * scale
    return ratio * t / (1 + (ratio - 1) * t) * num_timesteps


class RFlow:
    def __init__(self, num_inference_steps: Optional[int] = None, num_train_steps: int = 1000, use_discrete_timesteps: bool = False,
                 use_timestep_transform: bool = True, sample_method: str = "logit-normal", cfg_scale: float = 4.0, loc: float = 0.0,
                 scale: float = 1.0, transform_scale: float = 1.0, **_):
        if sample_method not in ("uniform", "logit-normal"):
            raise ValueError("sample_method must be uniform or logit-normal")
        if use_discrete_timesteps and sample_method != "uniform":
            raise ValueError("discrete timesteps need uniform sampling")
        self.num_sampling_steps, self.num_timesteps = num_inference_steps, num_train_steps
        self.discrete, self.transform, self.method = use_discrete_timesteps, use_timestep_transform, sample_method
        self.cfg_scale, self.loc, self.scale, self.transform_scale = cfg_scale, loc, scale, transform_scale

    def _transform(self, t, model_kwargs, scale=1.0):
        if not self.transform or not model_kwargs or "height" not in model_kwargs:
            return t
        return resolution_timestep_transform(t, model_kwargs["height"].to(t.device), model_kwargs["width"].to(t.device),
                                             model_kwargs["num_frames"].to(t.device), scale=scale, num_timesteps=self.num_timesteps)

    def add_noise(self, x0, noise, t):
        s = _bcast(t.float() / self.num_timesteps, x0)
        return ((1 - s) * x0.float() + s * noise.float()).to(x0.dtype)

    def q_sample(self, x_start, noise=None, t=None, mask=None, model_kwargs=None, generator=None, **_):
        B = x_start.shape[0]
        if t is None:
            if self.discrete:
                t = torch.randint(0, self.num_timesteps, (B,), generator=generator).float()
            else:
                u = density_sample("uniform" if self.method == "uniform" else "logit_normal", B, self.loc, self.scale,
                                   generator=generator)
                t = u * self.num_timesteps
            t = self._transform(t.to(x_start.device), model_kwargs, self.transform_scale)
        if noise is None:
            noise = randn_like(x_start, generator)
        x_t = self.add_noise(x_start, noise, t)
        if mask is not None:                       # frames outside the mask stay clean
            x_t = torch.where(mask[:, None, :, None, None].bool(), x_t, x_start)
        return x_t, noise, t

    @staticmethod
    def training_losses(model_output, x_start, noise=None, t=None, mask=None, weights=None, **_):
        C = x_start.shape[1]
        v = model_output[:, :C] if model_output.shape[1] == 2 * C else model_output
        err = (v.float() - (x_start.float() - noise.float())) ** 2
        if weights is not None:
            err = err * _bcast(weights.to(err.device)[t.long()], err)
        return mean_flat(err, mask)

    @torch.no_grad()
    def sample(self, model: Callable, latents, model_kwargs=None, guidance_scale=None, mask=None, generator=None, **_):
        g = self.cfg_scale if guidance_scale is None else guidance_scale
        model_kwargs = dict(model_kwargs or {})
        B, n = latents.shape[0], self.num_sampling_steps
        ts = [self._transform(torch.full((B,), (1.0 - i / n) * self.num_timesteps, device=latents.device), model_kwargs)
              for i in range(n)]
        if self.discrete:
            ts = [t.round() for t in ts]
        C = latents.shape[1]
        added = mask.bool().clone() if mask is not None else None
        x = latents
        for i, t in enumerate(ts):
            if mask is not None:
                upper = (mask * self.num_timesteps) >= t[:, None]
                x0 = x.clone()
                noisy, _, _ = self.q_sample(x0, noise=randn_like(x0, generator), t=t)
                x = torch.where((upper & ~added)[:, None, :, None, None], noisy, x0)
                added = upper
                model_kwargs["video_mask"] = upper.repeat(2, 1)
            out = model(torch.cat([x, x]), torch.cat([t, t]), **model_kwargs)[:, :C]
            cond, uncond = out.chunk(2)
            v = uncond + g * (cond - uncond)
            dt = (ts[i] - ts[i + 1] if i + 1 < n else ts[i]) / self.num_timesteps
            x_new = (x.float() + v.float() * _bcast(dt, x)).to(latents.dtype)
            x = torch.where(upper[:, None, :, None, None], x_new, x0) if mask is not None else x_new
        return x


# ------------------------------------------------------------------------------------------------- discrete flow match
class FlowMatchDiscreteScheduler:
    def __init__(self, num_train_timesteps: int = 1000, num_inference_timesteps: Optional[int] = None, shift: float = 1.0,
                 reverse: bool = True, solver: str = "euler", sample_method: str = "logit_normal", logit_mean: float = 0.0,
                 logit_std: float = 1.0, precondition_outputs: bool = False, guidance_scale: float = 6.0,
                 guidance_rescale: float = 0.0, embedded_guidance_scale: Optional[float] = None, **_):
        if solver != "euler":
            raise ValueError("only the euler solver exists")
        self.T, self.num_inference_timesteps, self.shift, self.reverse = num_train_timesteps, num_inference_timesteps, shift, reverse
        self.sample_method, self.logit_mean, self.logit_std = sample_method, logit_mean, logit_std
        self.precondition_outputs = precondition_outputs
        self.guidance_scale, self.guidance_rescale, self.embedded_guidance_scale = guidance_scale, guidance_rescale, embedded_guidance_scale
        s = torch.linspace(1, 0, num_train_timesteps + 1)
        self.sigmas = s if reverse else s.flip(0)
        self.timesteps = self.sigmas[:-1] * num_train_timesteps

    def time_shift(self, s):
        return self.shift * s / (1 + (self.shift - 1) * s)

    def set_timesteps(self, num_inference_steps: int, device=None):
        s = self.time_shift(torch.linspace(1, 0, num_inference_steps + 1))
        self.sigmas = (s if self.reverse else 1 - s).to(device)
        self.timesteps = (self.sigmas[:-1] * self.T).to(torch.float32)
        self.num_inference_timesteps = num_inference_steps

    def _sample_indices(self, B, generator):
        u = density_sample(self.sample_method, B, self.logit_mean, self.logit_std, generator=generator)
        return (u * self.T).long().clamp(max=self.T - 1)

    def q_sample(self, x_start, t=None, noise=None, generator=None, **_):
        if noise is None:
            noise = randn_like(x_start, generator)
        if t is None:
            idx = self._sample_indices(x_start.shape[0], generator)
            t = self.timesteps[idx].to(x_start.device)
        sig = _bcast(t.float() / self.T, x_start)
        return ((1 - sig) * x_start.float() + sig * noise.float()).to(x_start.dtype), noise, t

    def training_losses(self, model_output, x_start=None, x_t=None, noise=None, mask=None, t=None, **_):
        if self.precondition_outputs:
            sig = _bcast(t.float() / self.T, model_output)
            model_output, target = model_output.float() * (-sig) + x_t.float(), x_start
        else:
            target = noise.float() - x_start.float()
        return ((model_output.float() - target.float()) ** 2).flatten(1).mean(1)

    def step(self, model_output, index: int, sample):
        dt = (self.sigmas[index + 1] - self.sigmas[index]).to(sample.device, torch.float32)
        return (sample.float() + model_output.float() * dt).to(sample.dtype)

    @torch.no_grad()
    def sample(self, model: Callable, latents, model_kwargs=None, negative_kwargs=None, num_inference_steps=None, **_):
        """Euler integration from sigma = 1 to 0.  ``negative_kwargs`` (the unconditional prompt) switches true
        classifier-free guidance on; ``embedded_guidance_scale`` is passed to distilled-guidance models as ``guidance``."""
        self.set_timesteps(num_inference_steps or self.num_inference_timesteps or 50, device=latents.device)
        model_kwargs = dict(model_kwargs or {})
        if self.embedded_guidance_scale is not None:
            model_kwargs["guidance"] = torch.full((latents.shape[0],), self.embedded_guidance_scale * 1000.0, device=latents.device)
        x = latents
        for i, t in enumerate(self.timesteps):
            tt = t.expand(x.shape[0]).to(x.device)
            out = model(x, tt, **model_kwargs)
            if negative_kwargs is not None and self.guidance_scale != 1.0:
                un = model(x, tt, **negative_kwargs)
                out = rescale_noise_cfg(un + self.guidance_scale * (out - un), out, self.guidance_rescale)
            x = self.step(out, i, x)
        return x


class HunyuanVideo15Scheduler(FlowMatchDiscreteScheduler):
    """Adds the training-time timestep sampler of HunyuanVideo-1.5: ``snr_type`` uniform / lognorm, then the same
    rational shift that inference uses (``train_shift``)."""

    def __init__(self, snr_type: str = "lognorm", train_shift: float = 1.0, **kw):
        kw.setdefault("sample_method", "logit_normal" if snr_type == "lognorm" else "uniform")
        super().__init__(**kw)
        self.train_shift = train_shift

    def q_sample(self, x_start, t=None, noise=None, generator=None, **_):
        if t is None:
            u = density_sample(self.sample_method, x_start.shape[0], self.logit_mean, self.logit_std, generator=generator)
            u = self.train_shift * u / (1 + (self.train_shift - 1) * u)
            t = (u * self.T).to(x_start.device)
        return super().q_sample(x_start, t=t, noise=noise, generator=generator)


# ------------------------------------------------------------------------------------------------- Open-Sora-Plan v1.5
def linear_quadratic_sigmas(num_steps: int, approximate_steps: int = 1000) -> torch.Tensor:
    """Decreasing sigmas 1 -> 0 on ``num_steps + 1`` points.  Measured from the clean end, the first half of the steps
    advances by 1 / approximate_steps each (as a fine ``approximate_steps`` grid would), the second half follows the
    parabola that continues that line with the same slope and reaches 1 at the last step."""
    if num_steps % 2 or approximate_steps % 2 or num_steps > approximate_steps:
        raise ValueError("num_steps and approximate_steps must be even, num_steps <= approximate_steps")
    h = num_steps // 2
    i = torch.arange(num_steps + 1, dtype=torch.float64)
    curve = (1.0 - num_steps / approximate_steps) / (num_steps - h) ** 2
    pos = i / approximate_steps + torch.where(i > h, curve * (i - h) ** 2, torch.zeros_like(i))
    return (1.0 - pos).float()


class OpenSoraPlanScheduler:
    def __init__(self, num_inference_steps: Optional[int] = None, guidance_scale: float = 4.5, guidance_rescale: float = 0.7,
                 use_linear_quadratic_schedule: bool = True, num_train_timesteps: int = 1000, shift: float = 1.0,
                 use_dynamic_shifting: bool = False, weighting_scheme: str = "logit_normal", logit_mean: float = 0.0,
                 logit_std: float = 1.0, mode_scale: float = 1.29, sigma_eps: Optional[float] = None, **_):
        self.num_inference_steps, self.guidance_scale, self.guidance_rescale = num_inference_steps, guidance_scale, guidance_rescale
        self.linear_quadratic, self.T, self.shift, self.dynamic = use_linear_quadratic_schedule, num_train_timesteps, shift, use_dynamic_shifting
        self.scheme, self.logit_mean, self.logit_std, self.mode_scale = weighting_scheme, logit_mean, logit_std, mode_scale
        self.sigma_eps = sigma_eps
        self.sigmas = None

    def sigma_shift(self, s, shift=None, gamma: float = 1.0):
        k = self.shift if shift is None else shift
        return k * s / (1 + (k - 1) * s) if gamma == 1.0 else k / (k + (1 / s - 1) ** gamma)

    def sample_sigmas(self, B, generator=None):
        s = density_sample(self.scheme, B, self.logit_mean, self.logit_std, self.mode_scale, generator)
        s = self.sigma_shift(s)
        if self.sigma_eps is not None:
            s = s.clamp(self.sigma_eps, 1 - self.sigma_eps)
        return s

    def loss_weight(self, sigmas):
        if self.scheme == "sigma_sqrt":
            return sigmas.float() ** -2.0
        if self.scheme == "cosmap":
            return 2.0 / (math.pi * (1 - 2 * sigmas + 2 * sigmas ** 2))
        return torch.ones_like(sigmas)

    def add_noise(self, x0, noise, sigmas):
        s = _bcast(sigmas, x0)
        return ((1 - s) * x0.float() + s * noise.float()).to(x0.dtype)

    def q_sample(self, x_start, noise=None, t=None, generator=None, **_):
        if noise is None:
            noise = randn_like(x_start, generator)
        sig = (self.sample_sigmas(x_start.shape[0], generator) if t is None else t.float() / self.T).to(x_start.device)
        return self.add_noise(x_start, noise, sig), noise, sig * self.T

    def training_losses(self, model_output, x_start, noise=None, t=None, mask=None, **_):
        w = _bcast(self.loss_weight(t.float() / self.T), model_output)
        return mean_flat(w * (model_output.float() - (noise.float() - x_start.float())) ** 2, mask)

    def set_sigmas(self, num_steps: int, device=None):
        if self.linear_quadratic:
            s = linear_quadratic_sigmas(num_steps, min(max(num_steps * 10, 250), 1000))
        else:
            s = self.sigma_shift(torch.linspace(1, 0, num_steps + 1))
        self.sigmas = s.to(device)
        return self.sigmas

    @torch.no_grad()
    def sample(self, model: Callable, latents, model_kwargs=None, negative_kwargs=None, num_inference_steps=None, **_):
        sig = self.set_sigmas(num_inference_steps or self.num_inference_steps or 50, latents.device)
        x = latents
        for i in range(len(sig) - 1):
            tt = (sig[i] * self.T).expand(x.shape[0])
            out = model(x, tt, **(model_kwargs or {}))
            if negative_kwargs is not None and self.guidance_scale > 1.0:
                un = model(x, tt, **negative_kwargs)
                out = rescale_noise_cfg(un + self.guidance_scale * (out - un), out, self.guidance_rescale)
            x = (x.float() + (sig[i + 1] - sig[i]) * out.float()).to(latents.dtype)
        return x


# ------------------------------------------------------------------------------------------------- CogVideoX
def zero_snr_alphas_cumprod_sqrt(num_timesteps: int = 1000, linear_start: float = 0.00085, linear_end: float = 0.012,
                                 shift_scale: float = 1.0, n: Optional[int] = None) -> torch.Tensor:
    """sqrt(alpha_bar) of the scaled-linear DDPM schedule, SNR-shifted by ``shift_scale`` and rescaled so the last step
    has exactly zero SNR.  Index 0 = cleanest step.  ``n`` < num_timesteps sub-samples evenly (last step kept)."""
    betas = torch.linspace(linear_start ** 0.5, linear_end ** 0.5, num_timesteps, dtype=torch.float64) ** 2
    ac = torch.cumprod(1 - betas, 0)
    ac = ac / (shift_scale + (1 - shift_scale) * ac)
    if n is not None and n < num_timesteps:
        idx = torch.linspace(num_timesteps - 1, 0, n).round().long().flip(0)
        ac = ac[idx]
    a = ac.sqrt()
    a0, aT = a[0].clone(), a[-1].clone()
    return ((a - aT) * a0 / (a0 - aT)).float()


class CogVideoDiffusion:
    def __init__(self, num_train_timesteps: int = 1000, shift_scale: float = 1.0, uniform_sampling: bool = False,
                 min_snr_value: Optional[float] = None, loss_type: str = "l2", offset_noise_level: float = 0.0,
                 num_inference_steps: int = 50, guidance_scale: float = 6.0, dynamic_cfg: bool = True, **_):
        if loss_type not in ("l1", "l2"):
            raise ValueError("loss_type must be l1 or l2")
        self.T, self.shift_scale, self.min_snr, self.loss_type = num_train_timesteps, shift_scale, min_snr_value, loss_type
        self.offset_noise_level, self.num_inference_steps = offset_noise_level, num_inference_steps
        self.guidance_scale, self.dynamic_cfg = guidance_scale, dynamic_cfg
        self.a_sqrt = zero_snr_alphas_cumprod_sqrt(num_train_timesteps, shift_scale=shift_scale)
        self.uniform_sampling = uniform_sampling

    def q_sample(self, x_start, noise=None, t=None, generator=None, rank: int = 0, world: int = 1, **_):
        """``uniform_sampling``: the T indices are split into ``world`` contiguous groups and rank r draws from group r,
        so one global batch covers the schedule evenly."""
        B = x_start.shape[0]
        if t is None:
            if self.uniform_sampling and world > 1:
                lo, hi = rank * self.T // world, (rank + 1) * self.T // world
                t = torch.randint(lo, max(hi, lo + 1), (B,), generator=generator)
            else:
                t = torch.randint(0, self.T, (B,), generator=generator)
        t = t.to(x_start.device).long()
        if noise is None:
            noise = randn_like(x_start, generator)
        if self.offset_noise_level > 0:
            noise = noise + _bcast(torch.randn(B, generator=generator), noise).to(noise.dtype) * self.offset_noise_level
        a = _bcast(self.a_sqrt.to(x_start.device)[t], x_start)
        x_t = a * x_start.float() + (1 - a ** 2).sqrt() * noise.float()
        return x_t.to(x_start.dtype), noise, t

    def denoise(self, model_output, x_t, t):
        """v-prediction -> x0: c_skip = sqrt(alpha_bar), c_out = -sqrt(1 - alpha_bar)."""
        a = _bcast(self.a_sqrt.to(x_t.device)[t.long()], x_t)
        return model_output.float() * (-(1 - a ** 2).sqrt()) + x_t.float() * a

    def training_losses(self, model_output, x_start, x_t=None, t=None, **_):
        a = _bcast(self.a_sqrt.to(x_start.device)[t.long()], x_start)
        w = 1.0 / (1 - a ** 2).clamp(min=1e-8)
        if self.min_snr is not None:
            w = w.clamp(max=self.min_snr)
        diff = self.denoise(model_output, x_t, t) - x_start.float()
        return (w * (diff ** 2 if self.loss_type == "l2" else diff.abs())).flatten(1).mean(1)

    @torch.no_grad()
    def sample(self, model: Callable, latents, model_kwargs=None, negative_kwargs=None, num_inference_steps=None, eta: float = 0.0,
               generator=None, **_):
        """Deterministic (eta = 0) DDIM walk over the zero-SNR schedule in v-prediction form; guidance follows the
        cosine ramp 1 + g (1 - cos(pi ((n - t) / n)^5)) / 2 when ``dynamic_cfg``."""
        n = num_inference_steps or self.num_inference_steps
        a_all = zero_snr_alphas_cumprod_sqrt(self.T, shift_scale=self.shift_scale, n=n).to(latents.device)
        idx = torch.linspace(self.T - 1, 0, n).round().long().flip(0)
        x = latents
        for k in reversed(range(n)):
            t = torch.full((x.shape[0],), int(idx[k]), device=x.device)
            v = model(x, t, **(model_kwargs or {}))
            if negative_kwargs is not None:
                g = self.guidance_scale
                if self.dynamic_cfg:
                    g = 1 + self.guidance_scale * (1 - math.cos(math.pi * ((n - 1 - k) / n) ** 5.0)) / 2
                un = model(x, t, **negative_kwargs)
                v = un + g * (v - un)
            a = a_all[k]
            s = (1 - a ** 2).clamp(min=0).sqrt()
            x0 = a * x.float() - s * v.float()
            eps = s * x.float() + a * v.float()
            if k == 0:
                x = x0.to(latents.dtype)
                break
            a_prev = a_all[k - 1]
            s_prev = (1 - a_prev ** 2).clamp(min=0).sqrt()
            x = (a_prev * x0 + s_prev * eps).to(latents.dtype)
        return x
