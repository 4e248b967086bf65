"""InternVL3 / InternVL3.5 against the Hugging Face ``internvl`` implementation on tiny configs: logits of a packed sample
with two image tiles (class token, absolute positions, layer scale, whole-width q/k norm, pixel shuffle, projector, Qwen2
or Qwen3 decoder), the weight map both ways, position restarts across packed sequences, a non-native tile size
(bicubic position table), and engine steps against plain autograd."""
import pytest
import torch

from mindspeed_mm_b200.checkpoint import hf as hfio
from mindspeed_mm_b200.models.internvl import InternVLConfig, InternVLModel, pixel_shuffle

transformers = pytest.importorskip("transformers")


def _hf_model(qwen3: bool, big_tower: bool, moe: bool = False):
    from transformers import InternVLConfig as HFConfig, InternVLForConditionalGeneration
    vis = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=[56, 56],
               patch_size=[14, 14], use_qk_norm=big_tower, norm_type="rms_norm" if big_tower else "layer_norm",
               attention_bias=not big_tower, use_mean_pooling=not big_tower, layer_norm_eps=1e-6)
    txt = dict(model_type="qwen3" if qwen3 else "qwen2", hidden_size=64, intermediate_size=128, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, vocab_size=160, rms_norm_eps=1e-6,
               rope_parameters=dict(rope_type="default", rope_theta=1e6))
    if qwen3:
        txt["head_dim"] = 16
    if moe:
        txt.update(model_type="qwen3_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                   decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
    cfg = HFConfig(vision_config=vis, text_config=txt, image_token_id=150, downsample_ratio=0.5)
    model = InternVLForConditionalGeneration(cfg)
    torch.manual_seed(0)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.randn_like(p) * (0.05 if p.dim() > 1 else 0.2) + (1.0 if p.dim() == 1 else 0.0))
    return model.eval().float()


def _load(hf, cfg):
    model = InternVLModel(cfg, ep_size=1).float()
    model.load_state_dict(hfio.to_internal(hf.state_dict(), hfio.internvl_ops(cfg, experts_fused=True)), strict=True)
    return model.eval()


def _sample(cfg, tiles=2, size=56):
    g = torch.Generator().manual_seed(1)
    per = (size // 14 // 2) ** 2
    ids = torch.cat([torch.randint(0, 140, (5,), generator=g), torch.full((tiles * per,), cfg.image_token_id),
                     torch.randint(0, 140, (7,), generator=g)])
    return ids, torch.randn(tiles, 3, size, size, generator=g)


@pytest.mark.parametrize("qwen3,big_tower,moe", [(True, False, False), (False, False, False), (True, True, False),
                                                 (True, False, True)])
def test_logits_match_transformers(qwen3, big_tower, moe):
    hf = _hf_model(qwen3, big_tower, moe)
    cfg = InternVLConfig.from_hf(hf.config.to_dict())
    tiny = InternVLConfig.tiny(qwen3=qwen3, big_tower=big_tower, moe=moe)
    assert cfg.vision == tiny.vision and cfg.text == tiny.text and cfg.tokens_per_tile == 4
    model = _load(hf, cfg)
    ids, pixels = _sample(cfg)
    T = ids.numel()
    with torch.no_grad():
        ref = hf(input_ids=ids[None], pixel_values=pixels, attention_mask=torch.ones_like(ids)[None]).logits[0]
        mine = model(dict(input_ids=ids, pixel_values=pixels, cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T))
    assert mine.shape == ref.shape
    assert (mine - ref).abs().max() <= 2e-4 * ref.abs().max().clamp_min(1.0), float((mine - ref).abs().max())


def test_resized_tile_and_packed_sequences():
    hf = _hf_model(True, False)
    cfg = InternVLConfig.from_hf(hf.config.to_dict())
    model = _load(hf, cfg)
    ids_a, px_a = _sample(cfg, tiles=1, size=84)             # 6 x 6 patches: the 4 x 4 position table is resized
    # transformers only resizes the table when asked through the tower; compare the tower + connector directly
    with torch.no_grad():
        tower = hf.model.vision_tower
        emb = tower.embeddings.patch_embeddings(px_a)
        emb = torch.cat([tower.embeddings.cls_token.expand(1, -1, -1), emb], dim=1)
        emb = emb + tower.embeddings.interpolate_pos_encoding(emb, 84, 84)
        hid = tower.layernorm(tower.encoder(emb).last_hidden_state)[:, 1:]
        want = hf.model.multi_modal_projector(hf.model.pixel_shuffle(hid.reshape(1, 6, 6, -1), 0.5).reshape(1, 9, -1))[0]
        got = model.image_features(px_a)
    assert (got - want).abs().max() <= 2e-4 * want.abs().max().clamp_min(1.0)
    # two packed sequences = the two sequences run on their own (positions restart, block-diagonal attention)
    ids_b, px_b = _sample(cfg, tiles=2, size=56)
    ids_c = torch.arange(3, 14)
    Tb, Tc = ids_b.numel(), ids_c.numel()
    with torch.no_grad():
        packed = model(dict(input_ids=torch.cat([ids_b, ids_c]), pixel_values=px_b,
                            cu_seqlens=torch.tensor([0, Tb, Tb + Tc], dtype=torch.int32), max_seqlen=max(Tb, Tc)))
        ref_b = hf(input_ids=ids_b[None], pixel_values=px_b).logits[0]
        ref_c = hf(input_ids=ids_c[None]).logits[0]
    ref = torch.cat([ref_b, ref_c])
    assert (packed - ref).abs().max() <= 2e-4 * ref.abs().max().clamp_min(1.0)


def test_pixel_shuffle_order():
    x = torch.arange(2 * 4 * 6 * 8, dtype=torch.float32).reshape(2, 4, 6, 8)
    from transformers import InternVLModel as HFModel
    want = HFModel.pixel_shuffle(None, x.clone(), 0.5)
    assert torch.equal(pixel_shuffle(x, 0.5), want)


def test_weight_map_round_trip():
    for qwen3, big in ((True, True), (False, False)):
        hf = _hf_model(qwen3, big)
        cfg = InternVLConfig.from_hf(hf.config.to_dict())
        ops = hfio.internvl_ops(cfg)
        src = {k: v.clone() for k, v in hf.state_dict().items()}
        back = hfio.to_hf(hfio.to_internal(src, ops), ops, modern_prefix=False)
        assert set(back) == set(src)
        for k in src:
            assert torch.equal(back[k], src[k]), k
    # MoE: the fused in-memory form and the per-expert form of published checkpoints give the same internal tensors
    hf = _hf_model(True, False, moe=True)
    cfg = InternVLConfig.from_hf(hf.config.to_dict())
    src = {k: v.clone() for k, v in hf.state_dict().items()}
    fused = hfio.to_internal(dict(src), hfio.internvl_ops(cfg, experts_fused=True))
    listed = {}
    for k, v in src.items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, dim=0)
                listed[k.replace("gate_up_proj", f"{e}.gate_proj.weight")] = g.clone()
                listed[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = u.clone()
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                listed[k.replace("down_proj", f"{e}.down_proj.weight")] = v[e].clone()
        else:
            listed[k] = v
    ops = hfio.internvl_ops(cfg)
    per_expert = hfio.to_internal(dict(listed), ops)
    assert set(per_expert) == set(fused)
    for k in fused:
        assert torch.equal(per_expert[k], fused[k]), k
    back = hfio.to_hf(per_expert, ops, modern_prefix=False)
    assert set(back) == set(listed) and all(torch.equal(back[k], listed[k]) for k in listed)


def test_engine_step_matches_autograd():
    from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig
    cfg = InternVLConfig.tiny(big_tower=True)
    ref = InternVLModel(cfg).float()
    ref.init_weights(0)
    with torch.device("meta"):
        net = InternVLModel(cfg)
    eng = FSDPEngine(net.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=1e-3))
    src = dict(ref.named_parameters())
    eng.materialize(lambda name, mod: [p.data.copy_(src[(name + "." if name else "") + k]) for k, p in mod.named_parameters()])
    ids, pixels = _sample(cfg)
    T = ids.numel()
    labels = torch.roll(ids, -1)
    labels[ids == cfg.image_token_id] = -100
    batch = dict(input_ids=ids, labels=labels, pixel_values=pixels, cu_seqlens=torch.tensor([0, T], dtype=torch.int32),
                 max_seqlen=T)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.0)
    for _ in range(2):
        opt.zero_grad()
        ls, n = ref(batch)
        (ls / n).backward()
        opt.step()
        eng.set_lr(1e-3)
        ls, n = net(batch, run=eng.run)
        (ls / n).backward()
        eng.end_micro_step()
        eng.finish_step()
    got = dict(eng.named_full_params())
    assert set(got) == set(src)
    for k, p in ref.named_parameters():
        assert torch.allclose(got[k], p, atol=2e-5), (k, float((got[k] - p).abs().max()))


def test_tile_processor_and_dataset(tmp_path):
    import json
    from mindspeed_mm_b200.data.internvl import (InternVLConversationDataset, InternVLTileProcessor, TilePackCollator,
                                                 closest_tile_grid, tile_grids)
    grids = tile_grids(1, 12)
    assert (1, 1) in grids and (3, 4) in grids and (12, 1) in grids and all(1 <= c * r <= 12 for c, r in grids)
    assert closest_tile_grid(2000, 1000, grids, 448) == (4, 2)         # 2:1 picture, large: the biggest 2:1 grid
    assert closest_tile_grid(200, 100, grids, 448) == (2, 1)           # small picture keeps the first 2:1 grid
    assert closest_tile_grid(300, 300, grids, 448) == (1, 1)
    proc = InternVLTileProcessor(image_size=56, max_tiles=6)
    img = torch.rand(3, 60, 170)
    tiles, grid = proc(img)
    assert tiles.shape == (4, 3, 56, 56) and grid == (4, 1, 4)          # 3 x 1 tiles + thumbnail
    whole = torch.nn.functional.interpolate(img[None], size=(56, 168), mode="bicubic", align_corners=False, antialias=True)[0]
    want = (whole.clamp(0, 1)[:, :, 56:112] - proc.mean[0]) / proc.std[0]
    assert torch.allclose(tiles[1], want, atol=1e-6)
    assert proc(torch.rand(3, 50, 50))[0].shape[0] == 1                 # one tile: no thumbnail

    cfg = InternVLConfig.tiny()                 # placeholder ids above the byte tokenizer's range (bytes + 6 specials)
    cfg.text.vocab_size, cfg.image_token_id, cfg.vision_start_token_id, cfg.vision_end_token_id = 320, 300, 298, 299
    recs = [dict(messages=[dict(role="user", content="<image>what is this?"), dict(role="assistant", content="a cat")],
                 images=["a"]),
            dict(messages=[dict(role="user", content="hello"), dict(role="assistant", content="hi there")])]
    path = tmp_path / "d.json"
    path.write_text(json.dumps(recs))

    class M:
        config = cfg
    ds = InternVLConversationDataset(model=M, files=[str(path)], processor=InternVLTileProcessor.for_config(cfg, max_tiles=4),
                                     image_loader=lambda p: torch.rand(3, 40, 90))
    a, b = ds[0], ds[1]
    n_tiles = a["pixel_values"].shape[0]
    assert n_tiles == 3 and a["pixel_values"].shape[1:] == (3, 56, 56)
    ids = a["input_ids"].tolist()
    first = ids.index(cfg.image_token_id)
    assert ids[first - 1] == cfg.vision_start_token_id and ids[first + n_tiles * 4] == cfg.vision_end_token_id
    assert ids.count(cfg.image_token_id) == n_tiles * cfg.tokens_per_tile
    assert (a["labels"] != -100).sum() > 0 and (a["labels"][: first + n_tiles * 4] == -100).all()
    assert b["pixel_values"].shape == (0, 3, 56, 56)
    batch = TilePackCollator.for_config(cfg)([a, b])
    T = batch["input_ids"].numel()
    assert batch["cu_seqlens"].tolist() == [0, len(ids), T] and batch["pixel_values"].shape[0] == 3
    assert batch["image_positions"].numel() == 12 and batch["labels"][len(ids) - 1] == -100
    model = InternVLModel(cfg).float()
    model.init_weights(0)
    loss_sum, n = model(batch)
    assert torch.isfinite(loss_sum) and int(n) == int((batch["labels"] != -100).sum())


def test_trainer_runs_the_internvl_recipe_on_image_files(tmp_path):
    """examples/internvl3.5/tiny_native.yaml on a json with two PNG files: tiles from the dataset, packed by the tile
    collator, three steps of the native trainer."""
    import json
    import os
    import numpy as np
    from PIL import Image
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    rng = np.random.default_rng(0)
    for name, (h, w) in (("a.png", (60, 150)), ("b.png", (80, 80))):
        Image.fromarray(rng.integers(0, 255, (h, w, 3), dtype=np.uint8)).save(tmp_path / name)
    recs = [dict(messages=[dict(role="user", content="<image>describe"), dict(role="assistant", content="wide picture")],
                 images=["a.png"]),
            dict(messages=[dict(role="user", content="<image>and this?"), dict(role="assistant", content="a square")],
                 images=["b.png"])]
    (tmp_path / "train.json").write_text(json.dumps(recs))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = load_config(os.path.join(root, "examples/internvl3.5/tiny_native.yaml"),
                       [f"data.dataset_param.basic_parameters.dataset=[{tmp_path}/train.json]",
                        f"data.dataset_param.basic_parameters.dataset_dir={tmp_path}"], world_size=1)
    tr = Trainer(args, device="cpu")
    assert type(tr.model).__name__ == "InternVLModel" and tr.model.config.image_token_id == 300
    hist = tr.train()
    losses = [h["loss"] for h in hist] if hist and isinstance(hist[0], dict) else list(hist)
    assert len(losses) == 3 and losses[-1] < losses[0]
