"""Gaussian (DDPM-family) diffusion: noise schedules, respacing, posterior, learned-variance loss, DDPM / DDIM samplers.

Covers the reference's ``DDPM`` (mindspeed_mm/models/diffusion/ddpm.py:30: epsilon / x0 prediction, fixed or learned-range
variance, MSE / rescaled-MSE / KL losses, timestep respacing), ``IDDPM`` (iddpm.py:19: DDIM sampling with classifier-free
guidance on the first three channels), and the helpers of ``diffusion_utils.py`` (beta schedules, ``space_timesteps``,
Gaussian KL, discretised log-likelihood).  Everything is a table lookup on tensors that live on the latent's device;
no Python-side per-sample loops.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Union

import torch


# ------------------------------------------------------------------------------------------------- schedules
def beta_schedule(name: str, n: int, beta_start: float = 1e-4, beta_end: float = 2e-2) -> torch.Tensor:
    """``linear`` (Ho et al., scaled to ``n``), ``scaled_linear`` (latent diffusion), ``cosine`` / ``squaredcos_cap_v2``."""
    if name == "linear":
        scale = 1000.0 / n
        return torch.linspace(scale * beta_start, scale * beta_end, n, dtype=torch.float64)
    if name == "scaled_linear":
        return torch.linspace(beta_start ** 0.5, beta_end ** 0.5, n, dtype=torch.float64) ** 2
    if name in ("cosine", "squaredcos_cap_v2"):
        t = torch.arange(n + 1, dtype=torch.float64) / n
        f = torch.cos((t + 0.008) / 1.008 * math.pi / 2) ** 2
        return (1 - f[1:] / f[:-1]).clamp(max=0.999)
    raise ValueError(f"unknown beta schedule {name!r}")


def space_timesteps(n_train: int, spec: Union[str, int, Sequence[int]]) -> List[int]:
    """Timesteps kept by a respacing spec: an int / "N" (N evenly spread steps), "ddimN" (fixed stride), or
    "a,b,c" (the schedule cut into equal sections with a, b, c steps each)."""
    if isinstance(spec, int):
        spec = str(spec)
    if isinstance(spec, str):
        if spec.startswith("ddim"):
            want = int(spec[4:])
            for stride in range(1, n_train):
                if len(range(0, n_train, stride)) == want:
                    return list(range(0, n_train, stride))
            raise ValueError(f"no integer stride gives {want} steps out of {n_train}")
        counts = [int(x) for x in spec.split(",")]
    else:
        counts = list(spec)
    if len(counts) == 1 and counts[0] >= n_train:
        return list(range(n_train))
    size, extra = divmod(n_train, len(counts))
    start, out = 0, []
    for i, c in enumerate(counts):
        sec = size + (1 if i < extra else 0)
        if c > sec:
            raise ValueError(f"cannot take {c} steps out of a section of {sec}")
        stride = 1.0 if c <= 1 else (sec - 1) / (c - 1)
        out += [start + round(stride * k) for k in range(c)]
        start += sec
    return sorted(set(out))


def normal_kl(mean1, logvar1, mean2, logvar2):
    return 0.5 * (-1.0 + logvar2 - logvar1 + torch.exp(logvar1 - logvar2) + (mean1 - mean2) ** 2 * torch.exp(-logvar2))


def _std_normal_cdf(x):
    return 0.5 * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def discretized_gaussian_log_likelihood(x, means, log_scales):
    """log-likelihood of data quantised to 256 bins in [-1, 1] under a Gaussian (the t = 0 decoder term)."""
    c = x - means
    inv = torch.exp(-log_scales)
    cdf_plus, cdf_min = _std_normal_cdf(inv * (c + 1.0 / 255.0)), _std_normal_cdf(inv * (c - 1.0 / 255.0))
    log_cdf_plus = torch.log(cdf_plus.clamp(min=1e-12))
    log_one_minus = torch.log((1.0 - cdf_min).clamp(min=1e-12))
    mid = torch.log((cdf_plus - cdf_min).clamp(min=1e-12))
    return torch.where(x < -0.999, log_cdf_plus, torch.where(x > 0.999, log_one_minus, mid))


def mean_flat(x, mask=None):
    """Mean over all non-batch dims; ``mask`` [B, T] selects frames of a [B, C, T, H, W] tensor."""
    if mask is None:
        return x.flatten(1).mean(1)
    m = mask[:, None, :, None, None].to(x.dtype)
    per_frame = x.shape[1] * x.shape[3] * x.shape[4]
    return (x * m).flatten(1).sum(1) / (mask.flatten(1).sum(1).clamp(min=1) * per_frame)


def randn_like(x: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Standard normal of ``x``'s shape / dtype / device; a CPU generator is honoured for CUDA tensors too (the draw is
    made on the host in fp32 and copied), so a seed gives the same noise on every device."""
    if generator is None:
        return torch.randn_like(x)
    dev = generator.device
    return torch.randn(x.shape, generator=generator, dtype=torch.float32, device=dev).to(x.device, x.dtype)


def randint(high: int, n: int, device, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    if generator is None:
        return torch.randint(0, high, (n,), device=device)
    return torch.randint(0, high, (n,), generator=generator, device=generator.device).to(device)


def _take(table: torch.Tensor, t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    v = table.to(like.device)[t.long()].to(torch.float32)
    return v.reshape(-1, *([1] * (like.dim() - 1)))


# ------------------------------------------------------------------------------------------------- DDPM / IDDPM
class GaussianDiffusion:
    def __init__(self, num_inference_steps: Optional[int] = None, num_train_steps: int = 1000,
                 timestep_respacing: Union[str, Sequence[int], None] = None, noise_schedule: str = "linear",
                 use_kl: bool = False, sigma_small: bool = False, predict_xstart: bool = False, learn_sigma: bool = True,
                 rescale_learned_sigmas: bool = False, prediction_type: Optional[str] = None, snr_gamma: Optional[float] = None,
                 cfg_scale: float = 4.0, cfg_channels: Optional[int] = 3, beta_start: float = 1e-4, beta_end: float = 2e-2, **_):
        self.num_train_steps = num_train_steps
        self.loss_type = "rescaled_kl" if use_kl else ("rescaled_mse" if rescale_learned_sigmas else "mse")
        self.mean_type = prediction_type or ("x0" if predict_xstart else "epsilon")        # epsilon | x0 | v
        self.var_type = "learned_range" if learn_sigma else ("fixed_small" if sigma_small else "fixed_large")
        self.snr_gamma, self.cfg_scale, self.cfg_channels = snr_gamma, cfg_scale, cfg_channels
        base = beta_schedule(noise_schedule, num_train_steps, beta_start, beta_end)
        if num_inference_steps is not None:
            timestep_respacing = str(num_inference_steps)
        keep = space_timesteps(num_train_steps, timestep_respacing if timestep_respacing else [num_train_steps])
        ac = torch.cumprod(1.0 - base, 0)
        kept_ac = ac[keep]
        prev = torch.cat([torch.ones(1, dtype=torch.float64), kept_ac[:-1]])
        self.betas = 1.0 - kept_ac / prev
        self.timestep_map = torch.tensor(keep, dtype=torch.float32)       # respaced index -> original timestep
        self.num_timesteps = len(keep)
        self.alphas_cumprod = kept_ac
        self.alphas_cumprod_prev = prev
        self.sqrt_ac = kept_ac.sqrt()
        self.sqrt_1m_ac = (1.0 - kept_ac).sqrt()
        self.sqrt_recip_ac = (1.0 / kept_ac).sqrt()
        self.sqrt_recipm1_ac = (1.0 / kept_ac - 1.0).sqrt()
        self.posterior_variance = self.betas * (1.0 - prev) / (1.0 - kept_ac)
        pv = self.posterior_variance
        self.posterior_log_variance = torch.log(torch.cat([pv[1:2], pv[1:]])) if len(pv) > 1 else torch.log(pv.clamp(min=1e-20))
        self.posterior_coef_x0 = self.betas * prev.sqrt() / (1.0 - kept_ac)
        self.posterior_coef_xt = (1.0 - prev) * (1.0 - self.betas).sqrt() / (1.0 - kept_ac)

    # ------------------------------------------------------------------------------------ forward process
    def q_sample(self, x_start, t=None, noise=None, generator=None, **_):
        if noise is None:
            noise = randn_like(x_start, generator)
        if t is None:
            t = randint(self.num_timesteps, x_start.shape[0], x_start.device, generator)
        x_t = _take(self.sqrt_ac, t, x_start) * x_start.float() + _take(self.sqrt_1m_ac, t, x_start) * noise.float()
        return x_t.to(x_start.dtype), noise, t

    def model_timesteps(self, t):
        """The timestep values the network sees (original, un-respaced numbering)."""
        return self.timestep_map.to(t.device)[t.long()]

    def q_posterior(self, x_start, x_t, t):
        mean = _take(self.posterior_coef_x0, t, x_t) * x_start.float() + _take(self.posterior_coef_xt, t, x_t) * x_t.float()
        return mean, _take(self.posterior_variance, t, x_t), _take(self.posterior_log_variance, t, x_t)

    def predict_xstart(self, x_t, t, out):
        if self.mean_type == "x0":
            return out.float()
        if self.mean_type == "v":
            return _take(self.sqrt_ac, t, x_t) * x_t.float() - _take(self.sqrt_1m_ac, t, x_t) * out.float()
        return _take(self.sqrt_recip_ac, t, x_t) * x_t.float() - _take(self.sqrt_recipm1_ac, t, x_t) * out.float()

    def predict_eps(self, x_t, t, x0):
        return (_take(self.sqrt_recip_ac, t, x_t) * x_t.float() - x0) / _take(self.sqrt_recipm1_ac, t, x_t)

    def p_mean_variance(self, model_output, x_t, t, clip_denoised: bool = False):
        C = x_t.shape[1]
        if self.var_type == "learned_range":
            out, frac = model_output[:, :C], (model_output[:, C:2 * C].float() + 1) / 2
            min_log = _take(self.posterior_log_variance, t, x_t)
            max_log = _take(torch.log(self.betas), t, x_t)
            log_var = frac * max_log + (1 - frac) * min_log
        else:
            out = model_output[:, :C]
            if self.var_type == "fixed_large":
                table = torch.log(torch.cat([self.posterior_variance[1:2], self.betas[1:]])) if self.num_timesteps > 1 \
                    else torch.log(self.betas)
            else:
                table = self.posterior_log_variance
            log_var = _take(table, t, x_t).expand_as(x_t)
        x0 = self.predict_xstart(x_t, t, out)
        if clip_denoised:
            x0 = x0.clamp(-1, 1)
        mean, _, _ = self.q_posterior(x0, x_t, t)
        return {"mean": mean, "log_variance": log_var, "pred_xstart": x0}

    # ------------------------------------------------------------------------------------ losses
    def _vb_terms_bpd(self, model_output, x_start, x_t, t, mask=None):
        true_mean, _, true_log_var = self.q_posterior(x_start, x_t, t)
        p = self.p_mean_variance(model_output, x_t, t)
        kl = mean_flat(normal_kl(true_mean, true_log_var, p["mean"], p["log_variance"]), mask) / math.log(2.0)
        nll = -mean_flat(discretized_gaussian_log_likelihood(x_start.float(), p["mean"], 0.5 * p["log_variance"]), mask) / math.log(2.0)
        return torch.where(t == 0, nll, kl)

    def training_losses(self, model_output, x_start, x_t=None, noise=None, mask=None, weights=None, t=None, **_):
        """Per-sample loss [B].  ``model_output`` has 2C channels when the variance is learned."""
        if self.loss_type == "rescaled_kl":
            return self._vb_terms_bpd(model_output, x_start, x_t, t) * self.num_timesteps
        C = x_start.shape[1]
        vb = None
        if self.var_type == "learned_range":
            frozen = torch.cat([model_output[:, :C].detach(), model_output[:, C:]], 1)
            vb = self._vb_terms_bpd(frozen, x_start, x_t, t, mask)
            if self.loss_type == "rescaled_mse":
                vb = vb * self.num_timesteps / 1000.0
            model_output = model_output[:, :C]
        if self.mean_type == "x0":
            target = x_start
        elif self.mean_type == "v":
            target = _take(self.sqrt_ac, t, x_start) * noise.float() - _take(self.sqrt_1m_ac, t, x_start) * x_start.float()
        else:
            target = noise
        err = (target.float() - model_output.float()) ** 2
        if weights is not None:
            err = err * _take(weights, t, err)
        if self.snr_gamma is not None:                                   # min-SNR-gamma weighting
            snr = self.alphas_cumprod / (1 - self.alphas_cumprod)
            capped = snr.clamp(max=self.snr_gamma)
            w = {"epsilon": capped / snr.clamp(min=1e-8), "v": capped / (snr + 1.0), "x0": capped}[self.mean_type]
            err = err * _take(w, t, err)
        mse = mean_flat(err, mask)
        return mse if vb is None else mse + vb

    # ------------------------------------------------------------------------------------ samplers
    def _guided(self, model: Callable, x, t, model_kwargs, guidance_scale):
        """Runs the network on [cond, uncond] halves and mixes the first ``cfg_channels`` channels."""
        if guidance_scale is None or guidance_scale == 1.0:
            return model(x, self.model_timesteps(t), **model_kwargs)
        out = model(torch.cat([x, x]), self.model_timesteps(torch.cat([t, t])), **model_kwargs)
        cond, uncond = out.chunk(2)
        k = self.cfg_channels if self.cfg_channels is not None else x.shape[1]
        mixed = uncond[:, :k] + guidance_scale * (cond[:, :k] - uncond[:, :k])
        return torch.cat([mixed, cond[:, k:]], 1)

    @torch.no_grad()
    def p_sample_loop(self, model: Callable, latents, model_kwargs=None, guidance_scale=None, clip_denoised=False, generator=None):
        model_kwargs = model_kwargs or {}
        x = latents
        for i in reversed(range(self.num_timesteps)):
            t = torch.full((x.shape[0],), i, device=x.device, dtype=torch.long)
            p = self.p_mean_variance(self._guided(model, x, t, model_kwargs, guidance_scale), x, t, clip_denoised)
            noise = randn_like(p["mean"], generator)
            x = (p["mean"] + (0.0 if i == 0 else 1.0) * torch.exp(0.5 * p["log_variance"]) * noise).to(latents.dtype)
        return x

    @torch.no_grad()
    def ddim_sample_loop(self, model: Callable, latents, model_kwargs=None, guidance_scale=None, eta: float = 0.0,
                         clip_denoised=False, generator=None):
        model_kwargs = model_kwargs or {}
        x = latents
        for i in reversed(range(self.num_timesteps)):
            t = torch.full((x.shape[0],), i, device=x.device, dtype=torch.long)
            p = self.p_mean_variance(self._guided(model, x, t, model_kwargs, guidance_scale), x, t, clip_denoised)
            eps = self.predict_eps(x, t, p["pred_xstart"])
            ab, ab_prev = _take(self.alphas_cumprod, t, x), _take(self.alphas_cumprod_prev, t, x)
            sigma = eta * torch.sqrt((1 - ab_prev) / (1 - ab)) * torch.sqrt(1 - ab / ab_prev)
            mean = p["pred_xstart"] * ab_prev.sqrt() + torch.sqrt((1 - ab_prev - sigma ** 2).clamp(min=0)) * eps
            if eta > 0 and i > 0:
                mean = mean + sigma * randn_like(mean, generator)
            x = mean.to(latents.dtype)
        return x

    def sample(self, model: Callable, latents, model_kwargs=None, guidance_scale=None, sampler: str = "ddpm", **kw):
        g = self.cfg_scale if guidance_scale is None else guidance_scale
        loop = self.ddim_sample_loop if sampler == "ddim" else self.p_sample_loop
        return loop(model, latents, model_kwargs, g, **kw)


class DDPM(GaussianDiffusion):
    """ddpm.py:30 -- ancestral sampling by default, no guidance channel split."""

    def __init__(self, **kw):
        kw.setdefault("cfg_channels", None)
        super().__init__(**kw)


class IDDPM(GaussianDiffusion):
    """iddpm.py:19 -- learned-range variance, DDIM sampling with guidance on the first three channels."""

    def __init__(self, num_inference_steps: Optional[int] = None, **kw):
        kw.setdefault("learn_sigma", True)
        super().__init__(num_inference_steps=num_inference_steps, **kw)

    def sample(self, model, latents, model_kwargs=None, guidance_scale=None, sampler: str = "ddim", **kw):
        return super().sample(model, latents, model_kwargs, guidance_scale, sampler, **kw)
