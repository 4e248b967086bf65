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


# ------------------------------------------------------------------------------------------------- Wan variants
def test_wan22_per_token_timesteps_match_uniform_when_equal():
    from mindspeed_mm_b200.models.wan_variants import Wan22Config, Wan22DiT
    torch.manual_seed(0)
    cfg = Wan22Config.tiny(per_token_timestep=True)
    m = Wan22DiT(cfg)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    lat = torch.randn(1, 16, 3, 4, 4)
    prompt = torch.randn(1, 16, 64)
    t = torch.tensor([400.0])
    uniform = m(lat, t, prompt)
    per_tok = m(lat, t[:, None].expand(1, 3 * 2 * 2), prompt)
    assert torch.allclose(uniform, per_tok, atol=1e-4)
    clean_first = m(lat, t, prompt, first_frame_clean=True)
    assert not torch.allclose(uniform, clean_first, atol=1e-4)
    tt = m.ti2v_timesteps(lat, t)
    assert tt.shape == (1, 12) and tt[0, :4].tolist() == [0, 0, 0, 0] and tt[0, 4:].tolist() == [400.0] * 8


def test_wan22_moe_ffn_and_expert_pair():
    from mindspeed_mm_b200.models.wan_variants import Wan22Config, Wan22DiT, WanExpertPair
    torch.manual_seed(0)
    m = Wan22DiT(Wan22Config.tiny(moe_num_experts=4, moe_top_k=2))
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    lat, prompt = torch.randn(1, 16, 2, 4, 4), torch.randn(1, 16, 64)
    out = m(lat, torch.tensor([100.0]), prompt)
    assert out.shape == lat.shape
    out.mean().backward()
    assert m.blocks[0].moe.gate_up.grad is not None and m.blocks[0].moe.router.weight.grad is not None
    assert not hasattr(m.blocks[0], "ffn_0")
    pair = WanExpertPair(Wan22Config.tiny())
    assert pair.expert_for(torch.tensor([900.0])) is pair.high_noise and pair.expert_for(torch.tensor([100.0])) is pair.low_noise
    lo, hi = pair.scheduler_boundaries("high")
    assert lo == 0.0 and abs(hi - 0.4167) < 1e-3
    assert abs(WanExpertPair(Wan22Config.tiny(model_type="i2v")).scheduler_boundaries("low")[0] - 0.357) < 1e-3
    names = [n for n, _ in pair.fsdp_units()]
    assert names[0].startswith("high_noise.") and names[-1].startswith("low_noise.")
    assert pair(lat, torch.tensor([900.0]), prompt).shape == lat.shape


def test_vace_hints_start_as_identity_and_train_only_the_branch():
    from mindspeed_mm_b200.models.wan import WanDiT
    from mindspeed_mm_b200.models.wan_variants import VaceConfig, VaceWanDiT
    torch.manual_seed(0)
    cfg = VaceConfig.tiny()
    m = VaceWanDiT(cfg)
    for n, p in m.named_parameters():
        if "after_proj" not in n and "before_proj" not in n:
            torch.nn.init.normal_(p, std=0.05)
    lat, prompt = torch.randn(1, 16, 2, 4, 4), torch.randn(1, 16, 64)
    ctrl = torch.randn(1, 20, 2, 4, 4)
    t = torch.tensor([300.0])
    base = m(lat, t, prompt)
    with_ctrl = m(lat, t, prompt, vace_context=ctrl)
    assert torch.allclose(base, with_ctrl, atol=1e-6)                 # zero-initialised projections: no effect at start
    torch.nn.init.normal_(m.vace_blocks[0].after_proj.weight, std=0.05)
    moved = m(lat, t, prompt, vace_context=ctrl, vace_scale=2.0)
    assert not torch.allclose(base, moved, atol=1e-5)
    m.freeze_trunk()
    moved = m(lat, t, prompt, vace_context=ctrl)
    moved.mean().backward()
    assert all((p.grad is None) == (not n.startswith("vace_")) or not p.requires_grad for n, p in m.named_parameters())
    assert m.vace_patch_embedding.weight.grad is not None and m.blocks[0].ffn_0.weight.grad is None


def test_generation_recipes_build_and_step_through_the_sora_wrapper():
    import json
    import os
    from mindspeed_mm_b200.models.diffusion import build_scheduler
    from mindspeed_mm_b200.models.registry import build_model
    from mindspeed_mm_b200.models.wan import SoRAModel
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for rel in ("wan2.2/pretrain_model_ti2v_tiny.json", "vace/pretrain_model_tiny.json", "cogvideox/pretrain_model_tiny.json",
                "opensoraplan/pretrain_model_tiny.json", "stepvideo/pretrain_model_tiny.json"):
        mm = json.load(open(os.path.join(root, "examples", rel)))
        torch.manual_seed(0)
        net = build_model(mm["predictor"]["model_id"], mm["predictor"])
        for p in net.parameters():
            torch.nn.init.normal_(p, std=0.05)
        model = SoRAModel(net, build_scheduler(mm["diffusion"]), seed=0)
        batch = dict(latents=torch.randn(2, 16, 2, 4, 4), prompt=torch.randn(2, 6, 64))
        loss = model(batch)
        assert loss.dim() == 0 and torch.isfinite(loss), rel
        loss.backward()
        assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in net.parameters()), rel
    big = json.load(open(os.path.join(root, "examples/wan2.2/pretrain_model_a14b_high_noise.json")))
    sched = build_scheduler(big["diffusion"])
    _, _, t = sched.q_sample(torch.zeros(1, 16, 1, 2, 2), generator=torch.Generator().manual_seed(0))
    assert float(t) >= 875.0                       # the high-noise expert only ever sees t above the boundary
