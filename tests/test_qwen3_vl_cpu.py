"""Qwen3-VL (dense and MoE) against the Hugging Face implementation on a tiny config: logits of a packed sample with one
image (interpolated position table, DeepStack injection, interleaved mRoPE, q/k norm, routed experts), the weight map
both ways, and generation with the key/value cache."""
import pytest
import torch

from mindspeed_mm_b200.checkpoint import hf as hfio
from mindspeed_mm_b200.models.qwen3_vl import Qwen3VLConfig, Qwen3VLModel, interleaved_mrope_cos_sin

transformers = pytest.importorskip("transformers")


def _hf_model(moe: bool):
    vis = dict(depth=3, hidden_size=128, intermediate_size=256, num_heads=4, out_hidden_size=256, num_position_embeddings=64,
               deepstack_visual_indexes=[0, 1], patch_size=16, spatial_merge_size=2, temporal_patch_size=2, in_channels=3,
               hidden_act="gelu_pytorch_tanh")
    txt = dict(num_hidden_layers=3, hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2,
               head_dim=64, vocab_size=32000, rms_norm_eps=1e-6,
               rope_parameters=dict(rope_type="default", rope_theta=5e6, mrope_section=[12, 10, 10], mrope_interleaved=True))
    ids = dict(image_token_id=31999, video_token_id=31998, vision_start_token_id=31997, vision_end_token_id=31996)
    if moe:
        from transformers.models.qwen3_vl_moe import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration
        txt.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, decoder_sparse_step=1, mlp_only_layers=[],
                   norm_topk_prob=True)
        cfg = Qwen3VLMoeConfig(vision_config=vis, text_config=txt, **ids)
        model = Qwen3VLMoeForConditionalGeneration(cfg)
    else:
        from transformers.models.qwen3_vl import Qwen3VLConfig as HFConfig, Qwen3VLForConditionalGeneration
        cfg = HFConfig(vision_config=vis, text_config=txt, **ids)
        model = Qwen3VLForConditionalGeneration(cfg)
    torch.manual_seed(0)
    with torch.no_grad():
        for p in model.parameters():            # HF leaves the fused experts / norms at constants: draw everything
            p.copy_(torch.randn_like(p) * (0.05 if p.dim() > 1 else 0.2) + (1.0 if p.dim() == 1 else 0.0))
    return model.eval().float()


def _sample(grid=(1, 6, 4)):
    t, h, w = grid
    n_img = t * h * w // 4
    g = torch.Generator().manual_seed(1)
    text_a = torch.randint(0, 30000, (5,), generator=g)
    text_b = torch.randint(0, 30000, (7,), generator=g)
    ids = torch.cat([text_a, torch.tensor([31997]), torch.full((n_img,), 31999), torch.tensor([31996]), text_b])
    pixels = torch.randn(t * h * w, 3 * 2 * 16 * 16, generator=g)
    return ids, pixels, torch.tensor([list(grid)])


@pytest.mark.parametrize("moe", [False, True])
def test_logits_match_transformers(moe):
    hf = _hf_model(moe)
    cfg = Qwen3VLConfig.tiny(moe=moe)
    model = Qwen3VLModel(cfg, ep_size=1).float()
    sd = hfio.to_internal(hf.state_dict(), hfio.qwen3vl_ops(cfg, experts_out_in=moe))
    missing, unexpected = model.load_state_dict(sd, strict=True)
    ids, pixels, grid = _sample()
    with torch.no_grad():
        types = (ids == cfg.image_token_id).int()[None]
        out = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=torch.ones_like(ids)[None],
                 mm_token_type_ids=types)
        pos_hf = hf.model.get_rope_index(ids[None], types, image_grid_thw=grid)[0][:, 0]
        pos, _ = cfg.rope_index(ids, grid)
        assert torch.equal(pos, pos_hf)
        T = ids.numel()
        batch = dict(input_ids=ids, position_ids=pos, pixel_values=pixels, image_grid_thw=grid,
                     cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
        mine = model(batch)
    ref = out.logits[0]
    assert mine.shape == ref.shape
    assert (mine - ref).abs().max() <= 2e-4 * ref.abs().max().clamp_min(1.0), float((mine - ref).abs().max())


def test_weight_map_round_trip():
    hf = _hf_model(True)
    cfg = Qwen3VLConfig.tiny(moe=True)
    ops = hfio.qwen3vl_ops(cfg, experts_out_in=True)
    src = {k: v.clone() for k, v in hf.state_dict().items()}
    back = hfio.to_hf(hfio.to_internal(src, ops), ops)
    assert set(back) == set(src)
    for k in src:
        assert torch.equal(back[k], src[k]), k


def test_interleaved_mrope_bands():
    pos = torch.stack([torch.full((4,), 1.0), torch.full((4,), 2.0), torch.full((4,), 3.0)])
    cos, _ = interleaved_mrope_cos_sin(pos, 64, 1e4, (12, 10, 10))
    inv = 1.0 / (1e4 ** (torch.arange(0, 64, 2).float() / 64))
    which = torch.ones(32)                      # temporal by default
    which[1:30:3], which[2:30:3] = 2.0, 3.0
    assert torch.allclose(cos[0, :32], torch.cos(which * inv), atol=1e-6)


def test_generation_cache_matches_rerun():
    from mindspeed_mm_b200.tasks.inference import VLMGenerator
    cfg = Qwen3VLConfig.tiny(moe=False)
    model = Qwen3VLModel(cfg, ep_size=1).float()
    model.init_weights(3)
    ids, pixels, grid = _sample()
    gen = VLMGenerator(model)
    a = gen.generate(ids, pixel_values=pixels, image_grid_thw=grid, max_new_tokens=5, use_cache=True)
    b = gen.generate(ids, pixel_values=pixels, image_grid_thw=grid, max_new_tokens=5, use_cache=False)
    assert torch.equal(a, b)


def test_trainer_loads_and_writes_a_transformers_checkpoint(tmp_path):
    """A checkpoint written by transformers' ``save_pretrained`` drives the native trainer (config.json -> model config,
    safetensors -> sharding engine), and the trainer's ``save_format: hf`` output loads back into transformers."""
    import os
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    hf = _hf_model(False)
    src = tmp_path / "hf_in"
    hf.save_pretrained(src, safe_serialization=True)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = load_config(os.path.join(root, "examples/qwen3vl/tiny_moe_native.yaml"),
                       ["model.model_id=qwen3_vl", f"model.model_name_or_path={src}", "parallel.expert_parallel_size=1",
                        "training.train_iters=1", "training.lr=0.0", f"training.save={tmp_path}/out", "training.save_format=hf",
                        "data.dataset_param.basic_parameters.seq_len=200", "data.dataloader_param.pin_memory=false"],
                       world_size=1)
    tr = Trainer(args, device="cpu")
    assert tr.model.config.text.num_experts == 0 and tr.model.config.vision.deepstack_visual_indexes == (0, 1)
    got = dict(tr.engine.named_full_params())
    want = hfio.to_internal(hf.state_dict(), hfio.qwen3vl_ops(tr.model.config))
    for k, v in want.items():
        assert torch.allclose(got[k].float(), v.float(), atol=1e-6), k
    tr.train()                                        # lr 0: weights unchanged, then the HF export runs
    from transformers.models.qwen3_vl import Qwen3VLForConditionalGeneration
    back = Qwen3VLForConditionalGeneration.from_pretrained(tmp_path / "out" / "hf", dtype=torch.float32)
    ref = hf.state_dict()
    for k, v in back.state_dict().items():
        assert torch.allclose(v, ref[k], atol=1e-6), k


def test_router_auxiliary_loss_gradient_is_attached_inside_the_blocks(monkeypatch):
    """``loss.backward()`` alone gives the gradients of ``loss + coef * mean_layers(aux)``: the MoE blocks attach the
    auxiliary term's gradient in their own backward (so it also flows when a unit is recomputed)."""
    from mindspeed_mm_b200.models.moe import SparseMoeBlock
    from mindspeed_mm_b200.parallel import ep as epmod
    cfg = Qwen3VLConfig.tiny(moe=True)
    cfg.text.router_aux_loss_coef = 0.1
    model = Qwen3VLModel(cfg, ep_size=1).float()
    model.init_weights(0)
    ids, pixels, grid = _sample()
    pos, _ = cfg.rope_index(ids, grid)
    T = ids.numel()
    labels = torch.cat([ids[1:], torch.tensor([-100])])
    batch = dict(input_ids=ids, labels=labels, position_ids=pos, pixel_values=pixels, image_grid_thw=grid,
                 cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    seen, orig = [], epmod.load_balancing_loss
    monkeypatch.setattr(epmod, "load_balancing_loss", lambda *a: seen.append(orig(*a)) or seen[-1])
    loss_sum, n = model(batch)
    (loss_sum / n).backward()
    attached = {k: p.grad.clone() for k, p in model.named_parameters() if p.grad is not None}
    assert float(model.aux_loss()) > 0
    model.zero_grad()
    seen.clear()
    for m in model.modules():
        if isinstance(m, SparseMoeBlock):
            m.aux_scale = 0.0
    loss_sum, n = model(batch)
    (loss_sum / n + 0.1 * torch.stack(seen).mean()).backward()
    for k, p in model.named_parameters():
        if p.grad is not None:
            assert torch.allclose(attached[k], p.grad, atol=1e-6, rtol=1e-4), k
    gate = [k for k in attached if k.endswith("mlp.gate.weight")]
    assert gate and all(attached[k].abs().max() > 0 for k in gate)


def test_lora_finetune_from_a_transformers_checkpoint_writes_peft_files(tmp_path):
    """LoRA on top of a transformers checkpoint through the native trainer: base weights land in the wrapped linears, only the
    adapters train, and the run leaves adapter_model.safetensors / adapter_config.json that load back into a second run."""
    import json
    import os
    from safetensors.torch import load_file
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    hf = _hf_model(False)
    src = tmp_path / "hf_in"
    hf.save_pretrained(src, safe_serialization=True)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    common = ["model.model_id=qwen3_vl", f"model.model_name_or_path={src}", "parallel.expert_parallel_size=1",
              "training.lr=1.0e-2", "training.lora.enable=true", "training.lora.rank=4", "training.lora.alpha=8",
              "training.lora.target_modules=[q_proj,v_proj,down_proj]", "data.dataset_param.basic_parameters.seq_len=200",
              "data.dataloader_param.pin_memory=false"]
    tr = Trainer(load_config(os.path.join(root, "examples/qwen3vl/tiny_moe_native.yaml"),
                             common + ["training.train_iters=2", f"training.save={tmp_path}/out"], world_size=1), device="cpu")
    got = dict(tr.engine.named_full_params())
    want = hfio.to_internal(hf.state_dict(), hfio.qwen3vl_ops(tr.model.config))
    assert torch.allclose(got["layers.0.qkv_proj.base.weight"], want["layers.0.qkv_proj.weight"], atol=1e-6)
    tr.train()
    after = dict(tr.engine.named_full_params())
    assert torch.equal(after["layers.0.qkv_proj.base.weight"], got["layers.0.qkv_proj.base.weight"])
    assert after["layers.0.qkv_proj.lora_B"].abs().max() > 0
    ad = tmp_path / "out" / "lora_adapter"
    peft = load_file(str(ad / "adapter_model.safetensors"))
    assert json.load(open(ad / "adapter_config.json"))["r"] == 4
    assert "base_model.model.model.language_model.layers.0.self_attn.q_proj.lora_B.weight" in peft
    tr2 = Trainer(load_config(os.path.join(root, "examples/qwen3vl/tiny_moe_native.yaml"),
                              common + ["training.train_iters=1", f"training.lora.pretrained_lora_path={ad}"], world_size=1),
                  device="cpu")
    again = dict(tr2.engine.named_full_params())
    assert torch.allclose(again["layers.0.qkv_proj.lora_B"], after["layers.0.qkv_proj.lora_B"])
