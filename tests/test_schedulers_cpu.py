"""Diffusion scheduler family: closed-form checks of the forward process, losses and samplers on toy problems."""
import math

import pytest
import torch

from mindspeed_mm_b200.models.diffusion import (DDPM, IDDPM, CogVideoDiffusion, DiffusionModel, FlowMatchDiscreteScheduler,
                                                HunyuanVideo15Scheduler, OpenSoraPlanScheduler, RFlow, build_scheduler)
from mindspeed_mm_b200.models.diffusion.flows import linear_quadratic_sigmas, zero_snr_alphas_cumprod_sqrt
from mindspeed_mm_b200.models.diffusion.gaussian import beta_schedule, normal_kl, space_timesteps


def test_space_timesteps_and_betas():
    assert space_timesteps(1000, "10") == [round(i * 999 / 9) for i in range(10)]
    assert space_timesteps(100, "ddim25") == list(range(0, 100, 4))
    assert len(space_timesteps(300, "10,15,20")) == 45
    assert space_timesteps(50, [50]) == list(range(50))
    b = beta_schedule("linear", 1000)
    assert abs(float(b[0]) - 1e-4) < 1e-9 and abs(float(b[-1]) - 2e-2) < 1e-9
    c = beta_schedule("cosine", 100)
    assert float(c.max()) <= 0.999 and (c > 0).all()
    assert float(normal_kl(torch.zeros(3), torch.zeros(3), torch.zeros(3), torch.zeros(3)).abs().max()) == 0


def test_ddpm_posterior_and_respacing_consistency():
    d = DDPM(num_train_steps=1000, learn_sigma=False)
    x0 = torch.randn(4, 3, 2, 4, 4)
    x_t, noise, t = d.q_sample(x0, t=torch.tensor([0, 10, 500, 999]))
    # epsilon prediction with the true noise recovers x0 exactly
    rec = d.predict_xstart(x_t, t, noise)
    assert torch.allclose(rec, x0, atol=2e-3)
    # respaced chain keeps the cumulative alphas of the steps it retains
    r = DDPM(num_train_steps=1000, timestep_respacing="50", learn_sigma=False)
    full = torch.cumprod(1 - beta_schedule("linear", 1000), 0)
    assert torch.allclose(r.alphas_cumprod, full[r.timestep_map.long()])
    assert r.num_timesteps == 50
    loss = d.training_losses(noise, x0, x_t=x_t, noise=noise, t=t)
    assert loss.shape == (4,) and float(loss.abs().max()) == 0


def test_iddpm_learned_sigma_loss_and_ddim_sampler_recovers_point_mass():
    d = IDDPM(num_inference_steps=20, num_train_steps=1000)
    x0 = torch.full((2, 3, 1, 2, 2), 0.3)
    x_t, noise, t = d.q_sample(x0, t=torch.tensor([3, 12]))
    out = torch.cat([noise, torch.zeros_like(noise)], 1).requires_grad_()
    loss = d.training_losses(out, x0, x_t=x_t, noise=noise, t=t)
    assert loss.shape == (2,) and torch.isfinite(loss).all()
    loss.sum().backward()
    assert out.grad[:, 3:].abs().sum() > 0 and out.grad[:, :3].abs().sum() == 0     # only the variance head sees the vb term

    # an oracle epsilon model for data concentrated at x0 makes DDIM land on x0
    def oracle(x, t_model, **kw):
        idx = torch.searchsorted(d.timestep_map, t_model.float().cpu()).to(x.device)
        a = d.sqrt_ac[idx].float().reshape(-1, 1, 1, 1, 1)
        s = d.sqrt_1m_ac[idx].float().reshape(-1, 1, 1, 1, 1)
        eps = (x - a * 0.3) / s
        return torch.cat([eps, torch.zeros_like(eps)], 1)

    out = d.sample(oracle, torch.randn(2, 3, 1, 2, 2), guidance_scale=1.0)
    assert torch.allclose(out, x0, atol=1e-3)


def test_v_prediction_and_min_snr():
    d = DDPM(num_train_steps=100, learn_sigma=False, prediction_type="v", snr_gamma=5.0)
    x0 = torch.randn(3, 2, 1, 2, 2)
    x_t, noise, t = d.q_sample(x0, t=torch.tensor([1, 50, 99]))
    a, s = d.sqrt_ac[t].float().reshape(-1, 1, 1, 1, 1), d.sqrt_1m_ac[t].float().reshape(-1, 1, 1, 1, 1)
    v = a * noise - s * x0
    assert torch.allclose(d.predict_xstart(x_t, t, v), x0, atol=1e-4)
    assert float(d.training_losses(v, x0, x_t=x_t, noise=noise, t=t).abs().max()) < 1e-10


def test_rflow_transform_and_sampler():
    r = RFlow(num_inference_steps=8, use_timestep_transform=True, sample_method="uniform")
    x0 = torch.randn(2, 4, 3, 4, 4)
    kw = {"height": torch.tensor([512, 1024]), "width": torch.tensor([512, 1024]), "num_frames": torch.tensor([1, 1])}
    x_t, noise, t = r.q_sample(x0, model_kwargs=kw, generator=torch.Generator().manual_seed(0))
    s = t / 1000
    assert torch.allclose(x_t, (1 - s).reshape(-1, 1, 1, 1, 1) * x0 + s.reshape(-1, 1, 1, 1, 1) * noise, atol=1e-5)
    # base resolution keeps t, 4x the area doubles the odds t / (1 - t)
    tt = r._transform(torch.tensor([500.0, 500.0]), kw)
    assert abs(float(tt[0]) - 500) < 1e-3 and abs(float(tt[1]) - 2 / 3 * 1000) < 1e-2
    loss = r.training_losses(x0 - noise, x0, noise=noise, t=t)
    assert float(loss.abs().max()) == 0
    # constant-velocity oracle: the Euler walk is exact
    target = torch.full_like(x0, 0.7)
    z = torch.randn_like(x0)
    out = r.sample(lambda x, t, **k: (target - z).repeat(2, 1, 1, 1, 1), z, model_kwargs={}, guidance_scale=1.0)
    assert torch.allclose(out, target, atol=1e-5)


def test_flow_match_discrete_and_hunyuan15():
    f = FlowMatchDiscreteScheduler(shift=7.0, num_inference_timesteps=10)
    f.set_timesteps(10)
    assert abs(float(f.sigmas[0]) - 1) < 1e-6 and float(f.sigmas[-1]) == 0
    mid = 0.5
    assert abs(float(f.time_shift(torch.tensor(mid))) - 7 * mid / (1 + 6 * mid)) < 1e-6
    x0 = torch.randn(3, 4, 2, 4, 4)
    g = torch.Generator().manual_seed(1)
    f2 = FlowMatchDiscreteScheduler()
    x_t, noise, t = f2.q_sample(x0, generator=g)
    sig = (t / 1000).reshape(-1, 1, 1, 1, 1)
    assert torch.allclose(x_t, (1 - sig) * x0 + sig * noise, atol=1e-5)
    assert float(f2.training_losses(noise - x0, x_start=x0, noise=noise, t=t).abs().max()) == 0
    p = FlowMatchDiscreteScheduler(precondition_outputs=True)
    assert float(p.training_losses(noise - x0, x_start=x0, x_t=x_t, noise=noise, t=t).abs().max()) < 1e-8
    z = torch.randn_like(x0)
    target = torch.zeros_like(x0) + 0.2
    out = f.sample(lambda x, t, **k: z - target, z, num_inference_steps=6)
    assert torch.allclose(out, target, atol=1e-5)
    h = HunyuanVideo15Scheduler(snr_type="uniform", train_shift=3.0)
    _, _, th = h.q_sample(x0, generator=torch.Generator().manual_seed(0))
    assert ((th >= 0) & (th <= 1000)).all()


def test_opensoraplan_schedule_and_weights():
    s = linear_quadratic_sigmas(10, 250)
    assert float(s[0]) == 1 and abs(float(s[-1])) < 1e-7 and (s[1:] < s[:-1]).all()
    assert abs(float(s[1]) - (1 - 1 / 250)) < 1e-6                 # linear half: one fine-grid step each
    o = OpenSoraPlanScheduler(weighting_scheme="cosmap", shift=2.0, sigma_eps=1e-3)
    sig = torch.tensor([0.25, 0.5])
    assert torch.allclose(o.loss_weight(sig), 2 / (math.pi * (1 - 2 * sig + 2 * sig ** 2)))
    x0 = torch.randn(2, 4, 2, 2, 2)
    x_t, noise, t = o.q_sample(x0, generator=torch.Generator().manual_seed(0))
    assert float(o.training_losses(noise - x0, x0, noise=noise, t=t).abs().max()) == 0
    z = torch.randn_like(x0)
    out = o.sample(lambda x, t, **k: z - 0.1, z, num_inference_steps=8)
    assert torch.allclose(out, torch.full_like(z, 0.1), atol=1e-5)


def test_cogvideo_zero_snr_and_sampler():
    a = zero_snr_alphas_cumprod_sqrt(1000)
    assert abs(float(a[-1])) < 1e-7 and (a[1:] <= a[:-1]).all()
    c = CogVideoDiffusion(num_inference_steps=25)
    x0 = torch.full((2, 4, 2, 2, 2), -0.4)
    x_t, noise, t = c.q_sample(x0, t=torch.tensor([5, 700]))
    al = c.a_sqrt[t].reshape(-1, 1, 1, 1, 1)
    v = al * noise - (1 - al ** 2).sqrt() * x0
    assert torch.allclose(c.denoise(v, x_t, t), x0, atol=1e-4)
    assert float(c.training_losses(v, x0, x_t=x_t, t=t).max()) < 1e-6

    def oracle(x, t, **k):                                         # v for data concentrated at x0
        al = c.a_sqrt[t.long()].reshape(-1, 1, 1, 1, 1)
        s = (1 - al ** 2).sqrt()
        eps = torch.where(s > 0, (x - al * x0) / s.clamp(min=1e-8), x)
        return al * eps - s * x0

    out = c.sample(oracle, torch.randn_like(x0))
    assert torch.allclose(out, x0, atol=1e-3)


def test_factory():
    s = build_scheduler({"model_id": "rflow", "num_inference_steps": 4})
    assert isinstance(s, RFlow)
    assert isinstance(DiffusionModel({"model_id": "iddpm", "num_inference_steps": 10}).get_model(), IDDPM)
    with pytest.raises(KeyError):
        build_scheduler({"model_id": "nope"})
