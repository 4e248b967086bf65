import torch

from mindspeed_mm_b200.api import stable_init_fn
from mindspeed_mm_b200.checkpoint import wan as wanck
from mindspeed_mm_b200.models.diffusion import FlowMatchScheduler
from mindspeed_mm_b200.models.wan import SoRAModel, WanConfig, WanDiT, sinusoidal_embedding
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig


def test_flow_match_schedule_shape():
    s = FlowMatchScheduler(num_train_timesteps=1000, shift=5, sigma_min=0.0, extra_one_step=True)
    assert len(s.sigmas) == 1000 and abs(float(s.sigmas[0]) - 1.0) < 1e-6
    # shifted sigma: s' = 5 s / (1 + 4 s)
    raw = torch.linspace(1.0, 0.0, 1001)[:-1]
    assert torch.allclose(s.sigmas, 5 * raw / (1 + 4 * raw))
    assert abs(float(s.weights.mean()) - 1.0) < 1e-4 and float(s.weights.min()) == 0.0
    x0, noise = torch.randn(1, 4, 2, 4, 4), torch.randn(1, 4, 2, 4, 4)
    xt, n, t = s.q_sample(x0, noise=noise, t=s.timesteps[300:301])
    sg = s.sigmas[300]
    assert torch.allclose(xt, (1 - sg) * x0 + sg * noise, atol=1e-6)
    # a perfect prediction has zero loss; Euler steps from pure noise with the exact velocity reach x0
    assert float(s.training_losses(noise - x0, x0, noise, t)) == 0.0
    inf = FlowMatchScheduler(num_inference_timesteps=20, shift=5, sigma_min=0.0, extra_one_step=True)
    out = inf.sample(lambda x, ts, p: noise - x0, noise.clone(), None)
    assert torch.allclose(out, x0, atol=1e-4)


def test_sinusoid_matches_definition():
    e = sinusoidal_embedding(torch.tensor([3.0]), 8)
    f = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -torch.arange(4, dtype=torch.float64) / 4)
    assert torch.allclose(e[0, :4].double(), (3.0 * f).cos(), atol=1e-6)


def _build(cfg, seed=0):
    with torch.device("meta"):
        net = WanDiT(cfg)
    model = SoRAModel(net, FlowMatchScheduler(shift=5, sigma_min=0.0, extra_one_step=True), seed=seed)
    eng = FSDPEngine(model.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=2e-3),
                     no_recompute=())
    eng.materialize(stable_init_fn(0.05, 0))
    return model, eng


def test_wan_trains_and_unpatchify_inverts_patchify():
    cfg = WanConfig.tiny()
    model, eng = _build(cfg)
    emb, head = model.predictor.embeddings, model.predictor.head
    x = torch.randn(2, 16, 2, 4, 6)
    tok, grid = emb.patchify(x)
    assert grid == (2, 2, 3) and tok.shape == (2, 12, 64)
    # the head emits patch pixels channel-last (pf, ph, pw, C) while the embedding reads them in Conv3d order
    tok_cl = tok.view(2, 12, 16, 1, 2, 2).permute(0, 1, 3, 4, 5, 2).reshape(2, 12, 64)
    assert torch.equal(head.unpatchify(tok_cl, grid), x)
    batch = dict(latents=torch.randn(1, 16, 3, 8, 8), prompt=torch.randn(1, 16, 64))
    losses = []
    for _ in range(6):
        model.generator.manual_seed(0)          # same noise / timestep every step: loss must go down
        eng.set_lr(2e-3)
        loss = model(batch, run=eng.run)
        loss.backward()
        eng.end_micro_step()
        eng.finish_step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0], losses


def test_wan_name_maps_roundtrip():
    cfg = WanConfig.tiny()
    cfg.model_type = "i2v"
    with torch.device("meta"):
        net = WanDiT(cfg)
    internal = {n: torch.randn(p.shape) for n, p in net.named_parameters()}
    mm_sd = wanck.internal_to_mm(internal)
    assert "blocks.0.self_attn.proj_q.weight" in mm_sd and "time_projection.1.weight" in mm_sd
    assert mm_sd["patch_embedding.weight"].dim() == 5 and "blocks.1.cross_attn.k_img.weight" in mm_sd
    hf = wanck.mm_to_diffusers(mm_sd)
    assert "blocks.0.attn1.to_q.weight" in hf and "scale_shift_table" in hf and "blocks.0.scale_shift_table" in hf
    assert "condition_embedder.time_proj.weight" in hf and "blocks.0.ffn.net.0.proj.weight" in hf
    back = wanck.mm_to_internal(wanck.diffusers_to_mm(hf))
    assert set(back) == set(internal)
    for k in internal:
        assert torch.equal(back[k], internal[k]), k
