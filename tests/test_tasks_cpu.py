import math

import torch

from mindspeed_mm_b200.api import stable_init_fn
from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel
from mindspeed_mm_b200.models.wan import WanConfig, WanDiT
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig
from mindspeed_mm_b200.tasks import evaluation as ev
from mindspeed_mm_b200.tasks import preference as pref
from mindspeed_mm_b200.tasks.inference import VLMGenerator, WanPipeline
from mindspeed_mm_b200.tasks.lora import apply_lora, lora_state_dict, merge_lora


class _L:
    rank, alpha, dropout = 4, 8, 0.0
    target_modules = ["q_proj", "o_proj", "visual.blocks.{*}.attn_proj"]


def _tiny():
    cfg = Qwen25VLConfig.tiny()
    cfg.text.num_layers = 1
    cfg.vision.depth = 1
    cfg.vision.fullatt_block_indexes = (0,)
    return cfg


def test_lora_trains_only_adapters_and_merges():
    from bench import make_batches
    cfg = _tiny()
    with torch.device("meta"):
        model = Qwen25VLModel(cfg)
    wrapped = apply_lora(model, _L)
    assert "layers.0.qkv_proj" in wrapped and "layers.0.o_proj" in wrapped and "visual.blocks.0.attn_proj" in wrapped
    eng = FSDPEngine(model.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=1e-2))
    eng.materialize(stable_init_fn(0.02, 0))
    before = {n: t.clone() for n, t in eng.named_full_params()}
    batch = make_batches(cfg, 1, 300, 1, 1, 224, 0, pin=False)[0]
    for _ in range(2):
        eng.set_lr(1e-2)
        ls, n = model(batch, run=eng.run)
        (ls / n).backward()
        eng.end_micro_step()
        eng.finish_step()
    after = dict(eng.named_full_params())
    changed = {n for n in before if not torch.equal(before[n], after[n])}
    assert changed and all("lora_" in n for n in changed), changed
    sd = lora_state_dict(eng.named_full_params())
    assert set(sd) == {n for n in before if "lora_" in n}
    merged = merge_lora({n: t.clone() for n, t in eng.named_full_params()}, _L.alpha / _L.rank)
    assert "layers.0.qkv_proj.weight" in merged and not any("lora" in k or ".base." in k for k in merged)
    w0, a, b = after["layers.0.o_proj.base.weight"], after["layers.0.o_proj.lora_A"], after["layers.0.o_proj.lora_B"]
    assert torch.allclose(merged["layers.0.o_proj.weight"], w0 + 2.0 * b @ a, atol=1e-6)


def test_vlm_generate_and_wan_pipeline():
    cfg = _tiny()
    with torch.device("meta"):
        model = Qwen25VLModel(cfg)
    eng = FSDPEngine(model.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32)
    eng.materialize(stable_init_fn(0.02, 0))
    gen = VLMGenerator(model, run=eng.run)
    out = gen.generate(torch.randint(0, 1000, (12,)), max_new_tokens=3)
    assert out.shape == (15,)
    # the key / value cache gives the tokens of the exact (re-run the whole prefix) decoding, with an image in the prompt
    from mindspeed_mm_b200.data.synthetic import SyntheticVLMDataset, SyntheticVLMSpec
    smp = SyntheticVLMDataset(SyntheticVLMSpec(seq_len=90, images_per_sample=1, image_size=112, vocab_size=cfg.text.vocab_size,
                                               image_token_id=cfg.image_token_id,
                                               vision_start_token_id=cfg.vision_start_token_id))[0]
    kw = dict(pixel_values=smp["pixel_values"], image_grid_thw=smp["image_grid_thw"], max_new_tokens=5)
    cached = gen.generate(smp["input_ids"], use_cache=True, **kw)
    exact = gen.generate(smp["input_ids"], use_cache=False, **kw)
    assert torch.equal(cached, exact) and cached.shape == (95,)
    wc = WanConfig.tiny()
    with torch.device("meta"):
        dit = WanDiT(wc)
    e2 = FSDPEngine(dit.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, no_recompute=())
    e2.materialize(stable_init_fn(0.02, 0))
    pipe = WanPipeline(dit, run=e2.run)
    pipe.scheduler.set_timesteps(3)
    vid = pipe(torch.randn(1, 16, 64), torch.zeros(1, 16, 64), frames=2, height=4, width=4)
    assert vid.shape == (1, 16, 2, 4, 4) and torch.isfinite(vid).all()


def test_preference_losses():
    pc, pr, rc, rr = torch.tensor([-1.0]), torch.tensor([-3.0]), torch.tensor([-2.0]), torch.tensor([-2.0])
    loss, cr, rj = pref.dpo_loss(pc, pr, rc, rr, beta=0.5)
    assert abs(float(loss) - (-math.log(1 / (1 + math.exp(-1.0))))) < 1e-6 and float(cr) == 0.5 and float(rj) == -0.5
    assert float(pref.dpo_loss(pc, pr, rc, rr, beta=0.5, loss_type="hinge")[0]) == 0.0
    adv = pref.grpo_advantages(torch.tensor([1.0, 2.0, 3.0, 10.0, 10.0, 13.0]), 3)
    assert abs(float(adv[:3].mean())) < 1e-6 and abs(float(adv[3:].mean())) < 1e-6
    l0 = pref.grpo_loss(torch.zeros(4), torch.zeros(4), torch.tensor([1.0, -1.0, 2.0, -2.0]))
    assert abs(float(l0)) < 1e-6                       # ratio 1: objective = -mean(adv) = 0
    lp = pref.sde_step_logprob(torch.zeros(2, 4), torch.zeros(2, 4), torch.zeros(2, 4), 0.8, 0.7)
    assert lp.shape == (2,) and torch.isfinite(lp).all()
    assert float(pref.bradley_terry_loss(torch.tensor([2.0]), torch.tensor([0.0]))) < math.log(2)
    lp_tok = torch.log(torch.tensor([0.5, 0.5, 0.25, 0.25, 0.25]))
    s = pref.sequence_logprobs(lp_tok, torch.tensor([1, -100, 1, 1, 1]), torch.tensor([0, 2, 5]))
    assert torch.allclose(s, torch.tensor([math.log(0.5), 3 * math.log(0.25)]))


def test_eval_metrics():
    assert ev.multiple_choice_match("The answer is (B).", "b") and not ev.multiple_choice_match("C", "B")
    assert ev.relaxed_accuracy("10.2", "10") and not ev.relaxed_accuracy("12", "10")
    assert ev.anls("hello wrld", ["hello world"]) > 0.8 and ev.anls("zzz", ["hello"]) == 0.0
    r = ev.evaluate(lambda s: s["guess"], [{"guess": "A", "answer": "A"}, {"guess": "B", "answer": "C"}], "multiple_choice")
    assert r == {"accuracy": 0.5, "n": 2}


def test_wan_i2v_condition_and_mmdit_pipeline():
    import torch
    from mindspeed_mm_b200.models.ae.wan_vae import WanVAE, WanVAEConfig
    from mindspeed_mm_b200.models.diffusion import FlowMatchScheduler
    from mindspeed_mm_b200.models.encoders import CLIPVisionConfig, CLIPVisionEncoder
    from mindspeed_mm_b200.models.mmdit import MMDiT, MMDiTConfig
    from mindspeed_mm_b200.tasks.inference import MMDiTPipeline, wan_i2v_condition
    torch.manual_seed(0)
    vae = WanVAE(WanVAEConfig.tiny()).eval()
    clip = CLIPVisionEncoder(CLIPVisionConfig.tiny()).eval()
    y, feat = wan_i2v_condition(torch.rand(1, 3, 32, 32) * 2 - 1, vae, clip, frames=9)
    assert y.shape == (1, 4 + 4, 3, 4, 4) and feat.shape == (1, 5, 64)
    assert y[0, :4, 0].min() == 1 and y[0, :4, 1:].max() == 0          # only the first latent frame is given

    cfg = MMDiTConfig.tiny()
    dit = MMDiT(cfg)
    for p in dit.parameters():
        torch.nn.init.normal_(p, std=0.02)
    pipe = MMDiTPipeline(dit, FlowMatchScheduler(num_inference_timesteps=3, shift=3.0, sigma_min=0.0, extra_one_step=True),
                         embedded_guidance=3.5)
    out = pipe(torch.randn(1, 6, cfg.text_dim), torch.randn(1, cfg.pooled_dim), frames=1, height=8, width=8,
               generator=torch.Generator().manual_seed(0))
    assert out.shape == (1, cfg.in_channels, 1, 8, 8) and torch.isfinite(out).all()


def test_posttrain_trainers_take_a_step():
    """Diffusion-DPO, flow-GRPO and VLM-DPO loops on toy models: losses are finite and parameters move."""
    import copy
    import torch
    from mindspeed_mm_b200.models.diffusion import FlowMatchScheduler
    from mindspeed_mm_b200.tasks.posttrain import DiffusionDPOTrainer, FlowGRPOTrainer, VLMDPOTrainer
    torch.manual_seed(0)

    class Vel(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.net = torch.nn.Conv3d(4, 4, 1)

        def forward(self, x, t, cond):
            return self.net(x) + cond.mean() * 0.0

    pol, ref = Vel(), Vel()
    ref.load_state_dict(pol.state_dict())
    opt = torch.optim.SGD(pol.parameters(), lr=1e-2)
    sch = FlowMatchScheduler(shift=3.0, sigma_min=0.0, extra_one_step=True)
    dpo = DiffusionDPOTrainer(pol, ref, sch, beta=10.0, optimizer=opt)
    w0 = pol.net.weight.detach().clone()
    r = dpo.train_step(dict(latents_win=torch.randn(2, 4, 2, 4, 4), latents_lose=torch.randn(2, 4, 2, 4, 4),
                            prompt=torch.randn(2, 3, 8)))
    assert abs(r["loss"] - 0.6931) < 1e-3            # policy == reference at the first step: -log sigmoid(0)
    assert not torch.equal(w0, pol.net.weight)

    grpo = FlowGRPOTrainer(pol, sch, reward_fn=lambda x, c: -x.flatten(1).pow(2).mean(1), group_size=4, num_steps=4,
                           clip_range=0.2, optimizer=opt)
    r = grpo.train_step(torch.randn(1, 3, 8), (4, 2, 4, 4))
    assert r["loss"] == r["loss"] and r["reward_std"] > 0

    class LM(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(32, 16)
            self.out = torch.nn.Linear(16, 32)

        def forward(self, batch):
            return self.out(self.emb(batch["input_ids"]))

    lm, lm_ref = LM(), LM()
    lm_ref.load_state_dict(lm.state_dict())
    ids = torch.randint(0, 32, (40,))
    labels = ids.roll(-1)
    labels[:5] = -100
    batch = dict(input_ids=ids, labels=labels, cu_seqlens=torch.tensor([0, 10, 20, 30, 40], dtype=torch.int32))
    vd = VLMDPOTrainer(lm, lm_ref, beta=0.1, optimizer=torch.optim.SGD(lm.parameters(), lr=1e-2))
    r = vd.train_step(batch)
    assert abs(r["loss"] - 0.6931) < 1e-3


def test_task_entry_points_on_tiny_configs(tmp_path):
    """inference / evaluation / post-training entry functions behind the root scripts."""
    import json
    import os
    import torch
    from mindspeed_mm_b200.runtime import task_entry as te
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = json.load(open(os.path.join(root, "examples", "wan2.1", "pretrain_model_tiny.json")))
    cfg.update(prompts=[[1, 2, 3]], frames=3, height=8, width=8, save_path=str(tmp_path))
    vids = te.inference_sora(cfg)
    assert vids[0].shape == (1, 16, 3, 8, 8) and os.path.exists(tmp_path / "sample_0000.pt")
    assert te.evaluate_gen(cfg)["num_samples"] == 1

    def pairs():
        while True:
            yield dict(latents_win=torch.randn(1, 16, 3, 8, 8), latents_lose=torch.randn(1, 16, 3, 8, 8),
                       prompt=torch.randn(1, 16, 64))
    assert abs(te.posttrain_sora_dpo(cfg, pairs(), steps=1)[0]["loss"] - 0.6931) < 1e-3
    r = te.posttrain_flux_dancegrpo({"predictor": {"preset": "tiny"}, "grpo": {"num_steps": 3, "group_size": 2}},
                                    [(torch.randn(1, 4, 32), torch.randn(1, 16))], lambda x, c: -x.flatten(1).pow(2).mean(1), steps=1)
    assert r[0]["reward_std"] > 0
    out = te.inference_vlm({"model": {"preset": "tiny"}, "prompts": [{"text": "hello"}], "max_new_tokens": 2})
    assert len(out) == 1
    (tmp_path / "q.jsonl").write_text(json.dumps({"question": "2+2?", "answer": "4"}) + "\n")
    res = te.evaluate_vlm({"dataset": str(tmp_path / "q.jsonl"), "metric": "exact_match"}, predict=lambda s: "4")
    assert list(res.values())[0] == 1.0 or res.get("accuracy", res.get("exact_match", 0)) == 1.0
    video = torch.rand(3, 4, 16, 16) * 2 - 1
    te.write_video(video, str(tmp_path / "v.mp4"), fps=4)
    assert os.path.getsize(tmp_path / "v.mp4") > 0


def test_ae_trainer_and_video_text_dataset(tmp_path):
    import json
    import numpy as np
    import torch
    from mindspeed_mm_b200.data.multimodal import VideoTextDataset, read_video_frames
    from mindspeed_mm_b200.models.ae.wan_vae import WanVAE, WanVAEConfig
    from mindspeed_mm_b200.runtime.task_entry import write_video
    from mindspeed_mm_b200.tasks.ae_train import AETrainer, NLayerDiscriminator3D, VAELoss
    torch.manual_seed(0)
    write_video(torch.rand(3, 9, 48, 64) * 2 - 1, str(tmp_path / "clip.mp4"), fps=8)
    (tmp_path / "d.jsonl").write_text(json.dumps({"path": "clip.mp4", "cap": "a test clip"}) + "\n")
    ds = VideoTextDataset(files=[str(tmp_path / "d.jsonl")], data_folder=str(tmp_path), num_frames=5, height=32, width=32,
                          text_len=16)
    s = ds[0]
    assert s["video"].shape == (3, 5, 32, 32) and s["prompt_ids"].shape == (16,) and int(s["prompt_mask"].sum()) == 11
    assert -1.0 <= float(s["video"].min()) and float(s["video"].max()) <= 1.0
    vae = WanVAE(WanVAEConfig.tiny())
    tr = AETrainer(vae, VAELoss(kl_weight=1e-4, disc_weight=0.5, disc_start=1),
                   NLayerDiscriminator3D(3, base=8, n_layers=2), lr=1e-3)
    video = s["video"][None]
    l0 = tr.train_step(video)
    l1 = tr.train_step(video)
    assert "d_loss" not in l0 and "d_loss" in l1 and "g_loss" in l1
    assert all(v == v for v in l1.values())


def test_feature_extraction_roundtrip_into_feature_dataset(tmp_path):
    import json
    import torch
    from mindspeed_mm_b200.data.multimodal import FeatureDataset, VideoTextDataset
    from mindspeed_mm_b200.models.towers import build_ae, build_text_encoder
    from mindspeed_mm_b200.runtime.task_entry import write_video
    from mindspeed_mm_b200.tasks.feature_extraction import extract_features
    torch.manual_seed(0)
    write_video(torch.rand(3, 9, 32, 32) * 2 - 1, str(tmp_path / "a.mp4"), fps=8)
    (tmp_path / "d.jsonl").write_text(json.dumps({"path": "a.mp4", "cap": "clip"}) + "\n")
    ds = VideoTextDataset(files=[str(tmp_path / "d.jsonl")], data_folder=str(tmp_path), num_frames=5, height=16, width=16, text_len=8)
    ae = build_ae({"model_id": "wan_video_vae", "base_dim": 8, "z_dim": 4, "dim_mult": [1, 2, 2, 2], "num_res_blocks": 1,
                   "latents_mean": [0] * 4, "latents_std": [1] * 4})
    te = build_text_encoder({"model_id": "UMT5", "vocab_size": 300, "d_model": 32, "d_kv": 8, "d_ff": 64, "num_layers": 1, "num_heads": 4})
    out = tmp_path / "feat"
    assert extract_features(ds, ae, te, str(out), i2v=True) == 1
    fd = FeatureDataset(index=str(out / "index_rank0.jsonl"), data_folder=str(out))
    s = fd[0]
    assert s["latents"].shape == (4, 2, 2, 2) and s["prompt"].shape == (8, 32) and s["first_frame_latents"].shape == (4, 1, 2, 2)


def test_text_to_video_pipeline_over_scheduler_families():
    import torch
    from mindspeed_mm_b200.models.diffusion import build_scheduler
    from mindspeed_mm_b200.models.video_dits import CrossDiT, JointDiT, VideoDiTConfig
    from mindspeed_mm_b200.tasks.inference import TextToVideoPipeline
    torch.manual_seed(0)
    dit = CrossDiT(VideoDiTConfig.tiny())
    for p in dit.parameters():
        torch.nn.init.normal_(p, std=0.05)
    text, neg = torch.randn(1, 5, 32), torch.zeros(1, 5, 32)
    for cfg in (dict(model_id="flow_match_discrete", shift=7.0, guidance_scale=3.0), dict(model_id="opensoraplan_v1_5", guidance_scale=2.0),
                dict(model_id="cogvideo_diffusion"), dict(model_id="rflow", num_inference_steps=3, use_timestep_transform=False),
                dict(model_id="iddpm", num_inference_steps=3, learn_sigma=False)):
        pipe = TextToVideoPipeline(dit, build_scheduler(cfg))
        kw = {} if cfg["model_id"] in ("rflow", "iddpm") else dict(num_inference_steps=4 if cfg["model_id"] != "opensoraplan_v1_5" else 4)
        out = pipe(text, neg, frames=2, height=4, width=4, generator=torch.Generator().manual_seed(0), **kw)
        assert out.shape == (1, 4, 2, 4, 4) and torch.isfinite(out).all(), cfg
    joint = JointDiT(VideoDiTConfig.tiny())
    for p in joint.parameters():
        torch.nn.init.normal_(p, std=0.05)
    pipe = TextToVideoPipeline(joint, preset="cogvideox", vae_decode=lambda z: z * 2)
    out = pipe(text, frames=2, height=4, width=4, generator=torch.Generator().manual_seed(0), num_inference_steps=3)
    assert out.shape == (1, 4, 2, 4, 4)


def test_lora_adapter_in_peft_layout_round_trip(tmp_path):
    """Adapters on fused projections are written per Hugging Face part (shared lora_A, own rows of lora_B): the files carry
    PEFT's names, un-fused modules with those adapters compute the same update, and the files load back."""
    import json
    import torch
    from safetensors.torch import load_file
    from types import SimpleNamespace
    from mindspeed_mm_b200.checkpoint import hf as hfio
    from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel
    from mindspeed_mm_b200.tasks.lora import apply_lora, from_peft_state, lora_state_dict, save_peft_adapter
    cfg = Qwen25VLConfig.tiny()
    cfg.text.num_layers, cfg.vision.depth, cfg.vision.fullatt_block_indexes = 1, 1, (0,)
    model = Qwen25VLModel(cfg).float()
    model.init_weights(0)
    lc = SimpleNamespace(rank=4, alpha=8, target_modules=["q_proj", "v_proj", "down_proj"], dropout=0.0)
    wrapped = apply_lora(model, lc)
    assert "layers.0.qkv_proj" in wrapped and "layers.0.down_proj" in wrapped
    torch.manual_seed(0)
    for n, p in model.named_parameters():
        if "lora_" in n:
            torch.nn.init.normal_(p, std=0.1)
    state = lora_state_dict(model.named_parameters())
    ops = hfio.qwen25vl_ops(cfg)
    save_peft_adapter(state, ops, str(tmp_path), lc, base_model="Qwen/Qwen2.5-VL-7B-Instruct")
    peft = load_file(str(tmp_path / "adapter_model.safetensors"))
    conf = json.load(open(tmp_path / "adapter_config.json"))
    assert conf["peft_type"] == "LORA" and conf["r"] == 4 and set(conf["target_modules"]) == {"q_proj", "k_proj", "v_proj", "down_proj"}
    t = cfg.text
    qb = peft["base_model.model.model.language_model.layers.0.self_attn.q_proj.lora_B.weight"]
    kb = peft["base_model.model.model.language_model.layers.0.self_attn.k_proj.lora_B.weight"]
    assert qb.shape == (t.num_attention_heads * t.head_dim, 4) and kb.shape == (t.num_key_value_heads * t.head_dim, 4)
    # per-part update == rows of the fused update
    a, b = state["layers.0.qkv_proj.lora_A"], state["layers.0.qkv_proj.lora_B"]
    fused = b @ a
    assert torch.allclose(qb @ peft["base_model.model.model.language_model.layers.0.self_attn.q_proj.lora_A.weight"],
                          fused[:qb.shape[0]])
    back = from_peft_state(peft, hfio.qwen25vl_ops(cfg))
    assert set(back) == set(state) and all(torch.equal(back[k], state[k]) for k in state)


def test_lora_on_a_mixture_of_experts_model_keeps_the_experts_frozen():
    """LoRA on the MoE recipe: adapters on the attention projections are the only trainable parameters; the fused
    experts (3-D tensors, their own sharding engine) stay frozen and untouched by the optimizer."""
    import os
    import torch
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = load_config(os.path.join(root, "examples/qwen3vl/tiny_moe_native.yaml"),
                       ["parallel.expert_parallel_size=1", "training.train_iters=2", "data.dataloader_param.pin_memory=false",
                        "training.lora.enable=true", "training.lora.rank=4", "training.lora.alpha=8",
                        "training.lora.target_modules=[qkv_proj,o_proj]"], world_size=1)
    tr = Trainer(args, device="cpu")
    before = {n: t.clone() for n, t in tr.engine.named_full_params()}
    tr.train()
    after = dict(tr.engine.named_full_params())
    moved = {n for n in before if not torch.equal(before[n], after[n])}
    assert moved and all("lora_" in n for n in moved), sorted(moved)[:5]
    assert any("experts" in n for n in before) and not any("experts" in n for n in moved)
