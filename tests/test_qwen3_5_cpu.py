"""Qwen3.5 (dense and MoE) against the Hugging Face implementation on a tiny config: logits of a packed sample with one
image through GDN layers, the gated full-attention layer with partial interleaved mRoPE, zero-centred norms and (MoE) the
shared expert; and the weight map both ways."""
import pytest
import torch

from mindspeed_mm_b200.checkpoint import hf as hfio
from mindspeed_mm_b200.models.qwen3_5 import Qwen35Config, Qwen35Model

transformers = pytest.importorskip("transformers")


def _hf_model(moe: bool):
    vis = dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, out_hidden_size=256, num_position_embeddings=64,
               patch_size=16, spatial_merge_size=2, temporal_patch_size=2, in_channels=3, hidden_act="gelu_pytorch_tanh")
    txt = dict(num_hidden_layers=4, hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2,
               head_dim=64, vocab_size=32000, rms_norm_eps=1e-6, linear_num_key_heads=2, linear_num_value_heads=4,
               linear_key_head_dim=32, linear_value_head_dim=32, linear_conv_kernel_dim=4,
               layer_types=["linear_attention"] * 3 + ["full_attention"],
               rope_parameters=dict(rope_type="default", rope_theta=1e7, partial_rotary_factor=0.25, mrope_section=[3, 3, 2],
                                    mrope_interleaved=True))
    ids = dict(image_token_id=31999, video_token_id=31998, vision_start_token_id=31997, vision_end_token_id=31996)
    if moe:
        from transformers.models.qwen3_5_moe import Qwen3_5MoeConfig, Qwen3_5MoeForConditionalGeneration
        txt.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=128)
        txt.pop("intermediate_size")
        model = Qwen3_5MoeForConditionalGeneration(Qwen3_5MoeConfig(vision_config=vis, text_config=txt, **ids))
    else:
        from transformers.models.qwen3_5 import Qwen3_5Config, Qwen3_5ForConditionalGeneration
        model = Qwen3_5ForConditionalGeneration(Qwen3_5Config(vision_config=vis, text_config=txt, **ids))
    torch.manual_seed(0)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.linspace(1.0, 4.0, p.numel())))
            elif p.dim() > 1:
                p.copy_(torch.randn_like(p) * 0.05)
            else:
                p.copy_(torch.randn_like(p) * 0.2)
    return model.eval().float()


def _sample(grid=(1, 6, 4)):
    t, h, w = grid
    n_img = t * h * w // 4
    g = torch.Generator().manual_seed(1)
    ids = torch.cat([torch.randint(0, 30000, (5,), generator=g), torch.tensor([31997]), torch.full((n_img,), 31999),
                     torch.tensor([31996]), torch.randint(0, 30000, (24,), generator=g)])
    return ids, torch.randn(t * h * w, 3 * 2 * 16 * 16, generator=g), torch.tensor([list(grid)])


@pytest.mark.parametrize("moe", [False, True])
def test_logits_match_transformers(moe):
    hf = _hf_model(moe)
    cfg = Qwen35Config.tiny(moe=moe)
    model = Qwen35Model(cfg, ep_size=1).float()
    sd = hfio.to_internal(hf.state_dict(), hfio.qwen35_ops(cfg, experts_out_in=moe))
    model.load_state_dict(sd, strict=True)
    ids, pixels, grid = _sample()
    with torch.no_grad():
        types = (ids == cfg.image_token_id).int()[None]
        ref = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=torch.ones_like(ids)[None],
                 mm_token_type_ids=types).logits[0]
        pos, _ = cfg.rope_index(ids, grid)
        T = ids.numel()
        mine = model(dict(input_ids=ids, position_ids=pos, pixel_values=pixels, image_grid_thw=grid,
                          cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T))
    assert mine.shape == ref.shape
    assert (mine - ref).abs().max() <= 3e-4 * ref.abs().max().clamp_min(1.0), float((mine - ref).abs().max())


@pytest.mark.parametrize("moe", [False, True])
def test_weight_map_round_trip(moe):
    hf = _hf_model(moe)
    cfg = Qwen35Config.tiny(moe=moe)
    src = {k: v.clone() for k, v in hf.state_dict().items()}
    back = hfio.to_hf(hfio.to_internal(src, hfio.qwen35_ops(cfg, experts_out_in=moe)), hfio.qwen35_ops(cfg, experts_out_in=moe))
    assert set(back) == set(src)
    for k in src:
        assert torch.allclose(back[k], src[k], atol=1e-6), k


def test_from_hf_config():
    hf = _hf_model(True)
    cfg = Qwen35Config.from_hf(hf.config.to_dict())
    t = cfg.text
    assert (t.num_layers, t.full_attention_interval, t.num_experts, t.shared_expert_intermediate_size) == (4, 4, 8, 128)
    assert t.partial_rotary_factor == 0.25 and tuple(t.mrope_section) == (3, 3, 2) and cfg.vision.deepstack_visual_indexes == ()


def test_multi_token_prediction_loss_and_shared_units_under_the_engine():
    """mtp_num_layers = 1: the extra loss equals the hand-computed one (next-next token, inside each packed sequence), and
    under the sharding engine (embedding and output head run twice per step, reduced after their last backward) the
    updated weights equal those of plain autograd + the same AdamW."""
    from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig
    from mindspeed_mm_b200.models.qwen3_5 import shift_in_sequences
    cfg = Qwen35Config.tiny()
    cfg.text.mtp_num_layers, cfg.text.num_layers, cfg.vision.depth = 1, 4, 1
    torch.manual_seed(0)
    ref = Qwen35Model(cfg, ep_size=1).float()
    ref.init_weights(1)
    ids = torch.randint(0, 30000, (50,))
    cu = torch.tensor([0, 20, 50], dtype=torch.int32)
    labels = shift_in_sequences(ids, cu, -100)
    assert labels[19] == -100 and labels[49] == -100 and labels[0] == ids[1]
    pos = torch.cat([torch.arange(20), torch.arange(30)]).expand(3, -1)
    batch = dict(input_ids=ids, labels=labels, position_ids=pos, cu_seqlens=cu, max_seqlen=30)
    loss_sum, n = ref(batch)
    main = float(loss_sum / n) - 0.1 * float(ref.last_mtp_losses[0])
    cfg0 = Qwen35Config.tiny()
    cfg0.text.num_layers, cfg0.vision.depth = 4, 1
    plain = Qwen35Model(cfg0, ep_size=1).float()
    plain.load_state_dict({k: v for k, v in ref.state_dict().items() if not k.startswith("mtp.")})
    ls0, n0 = plain(batch)
    assert abs(main - float(ls0 / n0)) < 1e-5 and float(ref.last_mtp_losses[0]) > 5.0
    # engine run vs plain autograd
    with torch.device("meta"):
        net = Qwen35Model(cfg, ep_size=1)
    eng = FSDPEngine(net.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=1e-3))
    src = dict(ref.named_parameters())
    eng.materialize(lambda name, mod: [p.data.copy_(src[(name + "." if name else "") + k]) for k, p in mod.named_parameters()])
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.0)
    for _ in range(2):
        opt.zero_grad()
        ls, nn_ = ref(batch)
        (ls / nn_).backward()
        opt.step()
        eng.set_lr(1e-3)
        ls, nn_ = net(batch, run=eng.run)
        (ls / nn_).backward()
        eng.end_micro_step()
        eng.finish_step()
    got = dict(eng.named_full_params())
    for k, p in ref.named_parameters():
        assert torch.allclose(got[k], p, atol=2e-5), (k, float((got[k] - p).abs().max()))
