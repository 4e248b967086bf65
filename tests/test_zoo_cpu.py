import pytest
import torch

from mindspeed_mm_b200.api import stable_init_fn
from mindspeed_mm_b200.models import registry
from mindspeed_mm_b200.models.diffusion import FlowMatchScheduler
from mindspeed_mm_b200.models.mmdit import MMDiT, MMDiTConfig, rope_nd
from mindspeed_mm_b200.models.qwen3_5 import Qwen35Config, Qwen35Model
from mindspeed_mm_b200.ops import reference as ref
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig


def test_registry_lists_builtin_models():
    registry._ensure_builtin()
    for name in ("qwen2_5vl", "qwen3_vl", "qwen3_vl_moe", "qwen3_5", "wandit", "hunyuanvideodit", "flux", "wan_flow_match_scheduler"):
        assert name in registry.model_register


def test_mmdit_trains():
    cfg = MMDiTConfig.tiny()
    with torch.device("meta"):
        net = MMDiT(cfg)
    eng = FSDPEngine(net.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=2e-3), no_recompute=())
    eng.materialize(stable_init_fn(0.05, 0))
    sch = FlowMatchScheduler(shift=3.0)
    x0, noise = torch.randn(2, 4, 2, 4, 4), torch.randn(2, 4, 2, 4, 4)
    txt, pooled = torch.randn(2, 5, 32), torch.randn(2, 16)
    xt, _, t = sch.q_sample(x0, noise=noise, t=sch.timesteps[400:401])
    losses = []
    for _ in range(5):
        eng.set_lr(2e-3)
        pred = net(xt, t.expand(2), txt, pooled, guidance=torch.full((2,), 3.5), run=eng.run)
        assert pred.shape == x0.shape
        loss = sch.training_losses(pred, x0, noise, t)
        loss.backward()
        eng.end_micro_step()
        eng.finish_step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]
    c, s = rope_nd((2, 2, 2), (4, 6, 6), 256.0)
    assert c.shape == (8, 8)


def test_qwen35_gdn_layer_is_causal_and_packed():
    from mindspeed_mm_b200.models.qwen3_5 import GatedDeltaNet
    cfg = Qwen35Config.tiny()
    torch.manual_seed(0)
    layer = GatedDeltaNet(cfg.text)
    for n, p in layer.named_parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, 0, 0.05)
    layer.post_init()
    x = torch.randn(40, cfg.text.hidden_size)
    cu = torch.tensor([0, 17, 40])
    y = layer(x, cu)
    x2 = x.clone()
    x2[30] += 1.0                               # a later token of sequence 1 ...
    y2 = layer(x2, cu)
    assert torch.allclose(y[:30], y2[:30], atol=1e-5)          # ... changes nothing before it
    x3 = x.clone()
    x3[5] += 1.0                                # a token of sequence 0 must not leak into sequence 1
    y3 = layer(x3, cu)
    assert torch.allclose(y[17:], y3[17:], atol=1e-5) and not torch.allclose(y[5:17], y3[5:17])


def _composable_batch(cfg):
    from mindspeed_mm_b200.data.collate import PackedVLMCollator
    from mindspeed_mm_b200.data.synthetic import SyntheticVLMDataset, SyntheticVLMSpec
    ds = SyntheticVLMDataset(SyntheticVLMSpec(seq_len=96, images_per_sample=1, image_size=56, vocab_size=1024,
                                              image_token_id=1023, vision_start_token_id=1021,
                                              temporal_patch=1 if cfg.vision_kind == "vit" else 2))
    b = PackedVLMCollator(1023, 1021, vit_head_dim=32)([ds[0], ds[1]])
    if cfg.vision_kind is None:
        b.pop("pixel_values")
    if cfg.audio is not None:
        b["audio_features"] = [torch.randn(16, 40)]
        b["input_ids"][5:15] = cfg.audio_token_id
    return b


def test_composable_presets_cover_the_reference_zoo_and_train():
    """Every remaining model id of the reference's zoo resolves to a switch setting that runs forward + backward
    with gradients on all parameters."""
    from mindspeed_mm_b200.models import zoo  # noqa: F401
    from mindspeed_mm_b200.models.composable import PRESETS, ComposableLM
    from mindspeed_mm_b200.models.registry import model_register
    for mid, cfg in PRESETS.items():
        assert mid in model_register
        torch.manual_seed(0)
        m = ComposableLM(cfg)
        m.init_weights(0)
        loss, n = m(_composable_batch(cfg))
        (loss / n).backward()
        # the line-break / separator vectors of tiled images only take part when a batch carries tile grids
        # (tests/test_anyres_cpu.py trains them)
        assert torch.isfinite(loss) and all(p.grad is not None for n_, p in m.named_parameters()
                                            if not n_.startswith("tile_format.")), mid


def test_composable_from_hf_config_switches():
    from mindspeed_mm_b200.models.composable import from_hf_config
    hf = {"model_type": "kimi_k2", "text_config": {
        "num_hidden_layers": 4, "hidden_size": 64, "num_attention_heads": 4, "vocab_size": 100, "kv_lora_rank": 16,
        "q_lora_rank": 24, "qk_nope_head_dim": 8, "qk_rope_head_dim": 8, "v_head_dim": 8, "n_routed_experts": 8,
        "num_experts_per_tok": 2, "moe_intermediate_size": 32, "n_shared_experts": 1, "first_k_dense_replace": 1},
        "vision_config": {"hidden_size": 32, "intermediate_size": 64, "num_hidden_layers": 2, "num_attention_heads": 2}}
    c = from_hf_config(hf)
    assert c.text.mixers == ("mla",) * 4 and c.text.ffns == ("dense", "moe", "moe", "moe")
    assert c.vision_kind == "vit" and c.text.shared_expert_intermediate_size == 32 and c.text.rope == "rope1d"


def test_ltx2_joint_audio_video_block():
    from mindspeed_mm_b200.models.ltx2 import LTX2Config, LTX2Model, fractional_rope
    torch.manual_seed(0)
    cfg = LTX2Config.tiny()
    m = LTX2Model(cfg)
    for p in m.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.05)
        else:
            torch.nn.init.normal_(p, std=0.02)
    for n, p in m.named_parameters():
        if n.endswith("q_norm") or n.endswith("k_norm"):
            torch.nn.init.ones_(p)
    B, Sv, Sa, L = 2, 12, 5, 7
    vpos = torch.stack([torch.arange(Sv) // 4, (torch.arange(Sv) // 2) % 2, torch.arange(Sv) % 2]).float()[None].expand(B, -1, -1)
    apos = torch.arange(Sa).float()[None, None].expand(B, -1, -1)
    vt = torch.full((B, Sv), 500.0)
    vt[:, :4] = 0.0                                                     # a clean conditioning frame
    args = dict(video_latent=torch.randn(B, Sv, 8), video_timesteps=vt, video_positions=vpos, context=torch.randn(B, L, 24),
                context_mask=torch.tensor([[1] * 7, [1] * 4 + [0] * 3]).bool(), video_target_velocity=torch.randn(B, Sv, 8),
                audio_latent=torch.randn(B, Sa, 6), audio_timesteps=torch.full((B, Sa), 300.0), audio_positions=apos,
                audio_target_velocity=torch.randn(B, Sa, 6), loss_mask=(vt > 0))
    out = m(**args)
    assert out["video_pred"].shape == (B, Sv, 8) and out["audio_pred"].shape == (B, Sa, 6) and torch.isfinite(out["loss"])
    out["loss"].backward()
    blk = m.transformer_blocks[0]
    assert blk.audio_to_video_attn.to_k.weight.grad is not None and blk.video_to_audio_attn.to_q.weight.grad is not None
    assert blk.scale_shift_table_a2v_ca_audio.grad is not None
    # padded context positions do not matter
    args2 = dict(args)
    ctx = args["context"].clone()
    ctx[1, 4:] += 10.0
    args2["context"] = ctx
    with torch.no_grad():
        a, b = m(**args)["video_pred"], m(**args2)["video_pred"]
    assert torch.allclose(a[1], b[1], atol=1e-5)
    # video-only call works and differs from the joint one (the audio stream feeds the video stream)
    with torch.no_grad():
        solo = m(**{k: v for k, v in args.items() if not k.startswith("audio")})
    assert solo["audio_pred"] is None and not torch.allclose(solo["video_pred"], a, atol=1e-5)
    cos, sin = fractional_rope(vpos, 16, 10000.0, (20, 2048, 2048))
    assert cos.shape == (B, Sv, 8) and torch.allclose(cos ** 2 + sin ** 2, torch.ones_like(cos), atol=1e-5)
    assert [n for n, _ in m.fsdp_units()][:3] == ["video_io", "audio_io", "transformer_blocks.0"]


def test_hunyuan_video_15_sparse_attention_path():
    from mindspeed_mm_b200.models.mmdit import HunyuanVideo15DiT, MMDiTConfig
    torch.manual_seed(0)
    base = dict(in_channels=4, out_channels=4, hidden_size=64, num_heads=4, num_double_blocks=2, text_dim=32, pooled_dim=16,
                rope_dims=(4, 6, 6))
    lat, txt, pooled = torch.randn(1, 4, 2, 4, 4), torch.randn(1, 4, 32), torch.randn(1, 16)
    t = torch.tensor([500.0])
    outs = {}
    for name, sp in (("dense", None), ("all", dict(tile=(1, 2, 2), kernel=(5, 5, 5), topk=1)), ("sparse", dict(tile=(1, 2, 2), kernel=(1, 1, 1), topk=1))):
        torch.manual_seed(1)
        m = HunyuanVideo15DiT(MMDiTConfig.hunyuan_video_15(sparse_attention=sp, **base))
        for p in m.parameters():
            torch.nn.init.normal_(p, std=0.05)
        outs[name] = m(lat, t, txt, pooled)
    assert outs["dense"].shape == lat.shape
    assert torch.allclose(outs["dense"], outs["all"], atol=1e-4)          # a window that covers the canvas is dense attention
    assert not torch.allclose(outs["dense"], outs["sparse"], atol=1e-4)
    full = MMDiTConfig.hunyuan_video_15()
    assert full.num_single_blocks == 0 and full.sparse_attention["tile"] == (6, 8, 8)


def test_video_dit_families():
    from mindspeed_mm_b200.models.registry import build_model
    from mindspeed_mm_b200.models.video_dits import (CrossDiT, JointDiT, VideoDiTConfig, grouped_self_attention, sparse_1d_groups)
    from mindspeed_mm_b200.ops import reference as R
    torch.manual_seed(0)
    g = sparse_1d_groups(10, 4, contiguous=False)
    assert g.shape == (4, 3) and g[0].tolist() == [0, 4, 8] and g[3].tolist() == [3, 7, -1]
    assert sparse_1d_groups(10, 4, contiguous=True)[0].tolist() == [0, 1, 2]
    q, k, v = (torch.randn(2, 10, 2, 8) for _ in range(3))
    o = grouped_self_attention(q, k, v, g)
    ref0 = R.attention_dense(q[:, [0, 4, 8]], k[:, [0, 4, 8]], v[:, [0, 4, 8]])
    ref3 = R.attention_dense(q[:, [3, 7]], k[:, [3, 7]], v[:, [3, 7]])
    assert torch.allclose(o[:, [0, 4, 8]], ref0, atol=1e-5) and torch.allclose(o[:, [3, 7]], ref3, atol=1e-5)
    lat, text, t = torch.randn(2, 4, 2, 4, 4), torch.randn(2, 5, 32), torch.tensor([10.0, 900.0])
    mask = torch.tensor([[1, 1, 1, 1, 1], [1, 1, 0, 0, 0]]).bool()

    def init(m):
        for p in m.parameters():
            torch.nn.init.normal_(p, std=0.05)
        return m

    for kw in (dict(), dict(sparse_n=2), dict(skip_connections=True, num_layers=4), dict(learn_sigma=True), dict(text_dim_2=12)):
        m = init(CrossDiT(VideoDiTConfig.tiny(**kw)))
        out = m(lat, t, text, mask, text_2=torch.randn(2, 1, 12) if kw.get("text_dim_2") else None)
        assert out.shape == (2, 8 if kw.get("learn_sigma") else 4, 2, 4, 4)
        out.mean().backward()
        if kw.get("skip_connections"):
            assert m.blocks[3].skip_proj.weight.grad is not None and m.blocks[0].skip_proj is None
    # masked text positions do not influence the result
    m = init(CrossDiT(VideoDiTConfig.tiny())).eval()
    text2 = text.clone()
    text2[1, 2:] += 5.0
    with torch.no_grad():
        assert torch.allclose(m(lat, t, text, mask)[1], m(lat, t, text2, mask)[1], atol=1e-5)
    j = init(JointDiT(VideoDiTConfig.tiny()))
    out = j(lat, t, text)
    assert out.shape == lat.shape
    out.mean().backward()
    assert j.blocks[0].ada.weight.grad is not None
    assert isinstance(build_model("satdit", dict(hidden_size=64, num_heads=4, num_layers=1, text_dim=32, in_channels=4, out_channels=4)), JointDiT)
    sparse = build_model("sparseummdit", dict(hidden_size=64, num_heads=4, num_layers=2, text_dim=32, in_channels=4, out_channels=4))
    assert isinstance(sparse, CrossDiT) and sparse.config.skip_connections and sparse.config.sparse_n == 4


def test_bagel_mot_routes_tokens_to_their_parameter_set():
    from mindspeed_mm_b200.models.omni import BagelConfig, BagelMoT, bagel_attention_mask
    torch.manual_seed(0)
    m = BagelMoT(BagelConfig.tiny())
    for n, p in m.named_parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.05)
        elif "norm" in n:
            torch.nn.init.ones_(p)
    # sample 0: 3 text, 2 vit, 3 text ; sample 1: 2 text, 4 latent tokens
    T = 14
    text_rows = torch.tensor([0, 1, 2, 5, 6, 7, 8, 9])
    batch = dict(input_ids=torch.randint(1, 100, (T,)), text_rows=text_rows, vit_rows=torch.tensor([3, 4]), vit_embeds=torch.randn(2, 24),
                 latent_rows=torch.tensor([10, 11, 12, 13]), latents=torch.randn(4, 16), latent_pos=torch.tensor([0, 1, 8, 9]),
                 timesteps=torch.full((4,), 0.4), noise=torch.randn(4, 16), position_ids=torch.cat([torch.arange(8), torch.arange(6)]),
                 cu_seqlens=torch.tensor([0, 8, 14], dtype=torch.int32), max_seqlen=8,
                 attention_masks=[bagel_attention_mask(["causal", "full", "causal"], [3, 2, 3]), bagel_attention_mask(["causal", "noise"], [2, 4])])
    labels = torch.full((T,), -100)
    labels[[0, 1, 5, 6, 8]] = torch.randint(0, 100, (5,))
    batch["labels"] = labels
    out = m(batch)
    assert torch.isfinite(out["loss"]) and out["ce"] is not None and out["mse"] is not None
    out["loss"].backward()
    l0 = m.layers[0]
    assert l0.und.qkv.weight.grad.abs().sum() > 0 and l0.gen.qkv.weight.grad.abs().sum() > 0
    assert m.io.vae2llm.weight.grad is not None and m.io.latent_pos_embed.grad[[0, 1, 8, 9]].abs().sum() > 0
    # text-only batch: the generation parameter set receives no gradient
    m.zero_grad()
    text_only = dict(input_ids=batch["input_ids"][:8], text_rows=torch.arange(8), labels=labels[:8].clone(), position_ids=torch.arange(8),
                     cu_seqlens=torch.tensor([0, 8], dtype=torch.int32), max_seqlen=8)
    text_only["labels"][3:5] = 7
    m(text_only)["loss"].backward()
    assert l0.gen.qkv.weight.grad is None or float(l0.gen.qkv.weight.grad.abs().sum()) == 0
    mask = bagel_attention_mask(["causal", "noise", "causal"], [2, 2, 2])
    assert mask[2, 3] and mask[3, 2] and not mask[4, 2] and mask[4, 0] and not mask[0, 1]


def test_reward_model_bradley_terry():
    from mindspeed_mm_b200.models.omni import RewardModelBT
    torch.manual_seed(0)
    rm = RewardModelBT()
    rm.backbone.init_weights()
    torch.nn.init.normal_(rm.value_head.rm_head.weight, std=0.1)
    T = 12
    batch = dict(input_ids=torch.randint(0, 1000, (T,)), position_ids=torch.cat([torch.arange(3), torch.arange(3), torch.arange(4), torch.arange(2)])[None].expand(3, -1),
                 cu_seqlens=torch.tensor([0, 3, 6, 10, 12], dtype=torch.int32), max_seqlen=4)
    r = rm.rewards(batch)
    assert r.shape == (4,)
    loss = rm(batch)
    loss.backward()
    assert rm.value_head.rm_head.weight.grad is not None and 0 <= float(rm.last_accuracy) <= 1
    assert "backbone.lm_head" not in [n for n, _ in rm.fsdp_units()]


def test_sdxl_unet_matches_published_size_and_trains_through_the_sora_wrapper():
    import json
    import os
    from mindspeed_mm_b200.models.diffusion import build_scheduler
    from mindspeed_mm_b200.models.registry import build_model
    from mindspeed_mm_b200.models.sdxl_unet import SDXLConfig, SDXLUNet, compute_time_ids
    from mindspeed_mm_b200.models.wan import SoRAModel
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    full = json.load(open(os.path.join(root, "examples/sdxl/pretrain_model.json")))
    with torch.device("meta"):
        big = build_model("sdxl_unet", full["predictor"])
    assert sum(p.numel() for p in big.parameters()) == 2_567_463_684          # the released SDXL-base denoiser
    tiny = json.load(open(os.path.join(root, "examples/sdxl/pretrain_model_tiny.json")))
    torch.manual_seed(0)
    net = build_model("sdxl_unet", tiny["predictor"])
    assert isinstance(net, SDXLUNet)
    sched = build_scheduler(tiny["diffusion"])
    assert abs(float(sched.betas[0]) - 0.00085) < 1e-9 and abs(float(sched.betas[-1]) - 0.012) < 1e-9
    model = SoRAModel(net, sched, seed=0)
    ids = compute_time_ids((64, 64), (0, 0), (64, 64))
    added = torch.cat([torch.randn(2, 24), ids[None].expand(2, -1)], 1)
    batch = dict(latents=torch.randn(2, 4, 1, 8, 8), prompt=torch.randn(2, 5, 48), added_cond=added)
    loss = model(batch)
    assert loss.dim() == 0 and torch.isfinite(loss)
    loss.backward()
    assert all(p.grad is not None for p in net.parameters())
    # the size conditioning is live: another crop offset changes the prediction
    x, t = torch.randn(1, 4, 8, 8), torch.tensor([500])
    a0 = torch.cat([torch.zeros(1, 24), compute_time_ids((64, 64), (0, 0), (64, 64))[None]], 1)
    a1 = torch.cat([torch.zeros(1, 24), compute_time_ids((64, 64), (16, 0), (64, 64))[None]], 1)
    p = torch.randn(1, 5, 48)
    assert (net(x, t, p, a0) - net(x, t, p, a1)).abs().max() > 0


def test_hunyuanvideo_checkpoint_names_round_trip():
    """Every parameter of the HunyuanVideo DiT (token refiner included) has a name in the published checkpoint layout;
    published -> internal -> published is the identity and loads strictly."""
    from mindspeed_mm_b200.checkpoint import hf as hfio
    from mindspeed_mm_b200.models.mmdit import HunyuanVideoDiT, MMDiTConfig
    import dataclasses
    cfg = dataclasses.replace(MMDiTConfig.tiny(), text_refiner_layers=2)
    torch.manual_seed(0)
    net = HunyuanVideoDiT(cfg)
    for p in net.parameters():
        torch.nn.init.normal_(p, std=0.05)
    ops = net.hf_ops()
    pub = hfio.to_hf({k: v.clone() for k, v in net.state_dict().items()}, ops, modern_prefix=False)
    assert pub["img_in.proj.weight"].shape == (64, 4, 1, 2, 2)
    for k in ("txt_in.individual_token_refiner.blocks.1.self_attn_qkv.weight", "txt_in.c_embedder.linear_2.bias",
              "double_blocks.0.img_attn_q_norm.weight", "double_blocks.0.txt_mlp.fc2.bias", "single_blocks.1.modulation.linear.weight",
              "single_blocks.0.linear1.weight", "final_layer.adaLN_modulation.1.bias", "guidance_in.mlp.2.weight"):
        assert k in pub, k
    assert not any(k.startswith("embed.") or ".mod.lin." in k for k in pub)
    back = hfio.to_internal(pub, net.hf_ops())
    twin = HunyuanVideoDiT(cfg)
    twin.load_state_dict(back, strict=True)
    lat, t = torch.randn(1, 4, 2, 8, 8), torch.tensor([400.0])
    txt, pooled, g = torch.randn(1, 6, 32), torch.randn(1, 16), torch.tensor([6.0])
    mask = torch.tensor([[True, True, True, True, False, False]])
    with torch.no_grad():
        a, b = net(lat, t, txt, pooled, g, txt_mask=mask), twin(lat, t, txt, pooled, g, txt_mask=mask)
        c = net(lat, t, txt, pooled, g)
    assert torch.equal(a, b) and not torch.allclose(a, c)          # the prompt mask matters


@pytest.mark.parametrize("recipe", ["glm4.5v", "kimi_k3", "kimik2_5", "magistral-2509", "mimov2_5", "step3_vl", "qwen3omni",
                                    "qwen3_asr", "funasr"])
def test_family_recipes_run_under_the_native_trainer(recipe):
    """examples/<family>/tiny_native.yaml: model id -> composable preset, synthetic samples shaped by that preset's vision
    tower (or none), packed collator, sharding engine with gradient clipping: two steps with a finite loss."""
    import math
    import os
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = load_config(os.path.join(root, "examples", recipe, "tiny_native.yaml"), ["training.train_iters=2"], world_size=1)
    tr = Trainer(args, device="cpu")
    hist = tr.train()
    losses = [float(h["loss"]) if isinstance(h, dict) else float(h) for h in hist]
    assert len(losses) == 2 and all(math.isfinite(x) for x in losses)
