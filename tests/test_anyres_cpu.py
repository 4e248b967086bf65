"""Any-resolution tiling: resolution choice, token layout, and the feature arrangement the model applies."""
import torch

from mindspeed_mm_b200.data import anyres
from mindspeed_mm_b200.data.anyres import AnyResSpec


def test_select_best_resolution_prefers_coverage_then_least_padding():
    cands = [(384, 384), (768, 384), (384, 768), (768, 768), (1152, 384)]
    assert anyres.select_best_resolution((800, 400), cands) == (768, 384)
    assert anyres.select_best_resolution((300, 900), cands) == (384, 768)
    assert anyres.select_best_resolution((100, 100), cands) == (384, 384)          # small pictures are not blown up past need
    assert anyres.select_best_resolution((2000, 2000), cands) == (768, 768)
    assert len(anyres.candidate_grid(384, 9)) == sum(1 for a in range(1, 10) for b in range(1, 10) if a * b <= 9)


def test_tile_views_cover_the_padded_picture():
    spec = AnyResSpec(image_size=32, patch_size=4, downsample_ratio=2, candidates=anyres.candidate_grid(32, 4))
    img = torch.rand(3, 30, 61)
    views, (tw, th) = anyres.tile_views(img, spec)
    assert (tw, th) == (2, 1) and views.shape == (3, 3, 32, 32)
    # local views stitched together give the padded picture; the pad colour is the mean -> zero after normalisation
    local = torch.cat([views[1], views[2]], 2)
    assert local.shape == (3, 32, 64) and torch.allclose(local[:, -1, :], torch.zeros(3, 64), atol=1e-6)
    assert anyres.image_token_count(spec, tw, th) == 4 * 5 + 1 + 4 * (8 + 1)
    v1, crop1 = anyres.tile_views(img, spec, cropping=False)
    assert crop1 == (1, 1) and v1.shape[0] == 2


def _encode(s):
    return [ord(c) % 200 for c in s]


def test_tokenize_with_images_and_sft_labels():
    spec = AnyResSpec(image_size=32, patch_size=4, downsample_ratio=2, candidates=anyres.candidate_grid(32, 4), image_token_id=1023)
    out = anyres.tokenize_with_images("ab<image>cd<image>e", [torch.rand(3, 32, 32), torch.rand(3, 64, 32)], _encode, spec,
                                      bos_id=1, eos_id=2)
    n0, n1 = out["num_image_tokens"]
    assert out["spatial_crop"].tolist() == [[1, 1], [1, 2]]
    assert n0 == 20 + 1 + 4 * 5 and n1 == 20 + 1 + 8 * 5
    assert out["input_ids"].numel() == 1 + 2 + n0 + 2 + n1 + 1 + 1
    assert int(out["images_seq_mask"].sum()) == n0 + n1 == int((out["input_ids"] == 1023).sum())
    assert out["views"].shape[0] == 2 + 3
    try:
        anyres.tokenize_with_images("no tag", [torch.rand(3, 8, 8)], _encode, spec)
        raise AssertionError("expected a tag / image count error")
    except ValueError:
        pass
    s = anyres.build_sft_sample([("<image>what?", "cat"), ("sure?", "yes")], [torch.rand(3, 32, 32)], _encode, spec, bos_id=1, eos_id=2)
    lab = s["labels"]
    assert lab.numel() == s["input_ids"].numel()
    kept = s["input_ids"][lab != -100].tolist()
    assert kept == _encode("cat") + [2] + _encode("yes") + [2]
    assert not bool((s["images_seq_mask"] & (lab != -100)).any())


def test_tile_formatter_layout_and_model_step():
    from mindspeed_mm_b200.models.composable import PRESETS, ComposableLM, TileFormatter
    # layout against a direct construction
    fmt = TileFormatter(4)
    with torch.no_grad():
        fmt.image_newline.fill_(-1.0)
        fmt.view_separator.fill_(-2.0)
    h = w = 2
    crops = torch.tensor([[2, 1]])
    feats = torch.arange(3 * h * w, dtype=torch.float32)[:, None].expand(-1, 4).contiguous()     # view v, cell k -> v * 4 + k
    got = fmt(feats, crops)[:, 0].tolist()
    glob = [0, 1, -1, 2, 3, -1]
    local = [4, 5, 8, 9, -1, 6, 7, 10, 11, -1]                  # row 0 of both tiles, then row 1
    assert got == glob + [-2] + local
    fmt.global_view_pos = "tail"
    assert fmt(feats, crops)[:, 0].tolist() == local + [-2] + glob

    cfg = PRESETS["deepseekvl2"]
    assert cfg.tile_format
    torch.manual_seed(0)
    model = ComposableLM(cfg)
    with torch.no_grad():
        model.init_weights(0)
    assert float(model.tile_format.image_newline.detach().abs().max()) < 0.5
    vit = cfg.vit
    spec = AnyResSpec(image_size=vit.patch_size * 4, patch_size=vit.patch_size, downsample_ratio=vit.merge,
                      candidates=anyres.candidate_grid(vit.patch_size * 4, 4), image_token_id=cfg.image_token_id)
    s = anyres.build_sft_sample([("<image>describe", "a wide photo")], [torch.rand(3, 40, 100)], _encode, spec, bos_id=1, eos_id=2)
    rows, grid = anyres.views_to_patch_rows(s["views"], vit.patch_size, vit.merge, vit.temporal_patch_size)
    T = s["input_ids"].numel()
    batch = dict(input_ids=s["input_ids"], labels=s["labels"], pixel_values=rows, image_grid_thw=grid,
                 spatial_crop=s["spatial_crop"], position_ids=torch.arange(T),
                 cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    out = model(batch)
    loss = out[0] / out[1] if isinstance(out, tuple) else out
    assert torch.isfinite(loss)
    loss.backward()
    assert model.tile_format.image_newline.grad.abs().sum() > 0 and model.tile_format.view_separator.grad.abs().sum() > 0


def test_tiled_dataset_and_pack_collator_feed_the_model(tmp_path):
    import json
    from mindspeed_mm_b200.data.anyres import TiledConversationDataset, TiledPackCollator
    from mindspeed_mm_b200.models.registry import data_register
    from mindspeed_mm_b200.models.composable import PRESETS, ComposableLM
    assert data_register.get("deepseekvl2") is TiledConversationDataset
    recs = [{"conversations": [{"from": "human", "value": "<image>\nwhat is this?"}, {"from": "gpt", "value": "a chart"}],
             "images": ["a.png"]},
            {"messages": [{"role": "user", "content": "hello"}, {"role": "assistant", "content": "hi there"}]}]
    (tmp_path / "d.json").write_text(json.dumps(recs))
    cfg = PRESETS["deepseekvl2"]
    torch.manual_seed(0)
    model = ComposableLM(cfg)
    with torch.no_grad():
        model.init_weights(0)

    class Tok:                                       # ids stay clear of the special ids at the top of the tiny vocabulary
        def encode(self, s):
            return [3 + ord(c) % 200 for c in s]

    ds = TiledConversationDataset(files=str(tmp_path / "d.json"), model=model, tokenizer=Tok(),
                                  image_loader=lambda p: torch.rand(3, 50, 120), bos_id=1, eos_id=2)
    assert len(ds) == 2
    a, b = ds[0], ds[1]
    assert a["spatial_crop"].shape == (1, 2) and b["spatial_crop"].shape == (0, 2) and b["views"].shape[0] == 0
    n_img = int(a["images_seq_mask"].sum())
    assert n_img == anyres.image_token_count(ds.spec, *a["spatial_crop"][0].tolist())
    batch = TiledPackCollator(cfg.vit.patch_size, cfg.vit.merge, cfg.vit.temporal_patch_size)([a, b])
    T = a["input_ids"].numel() + b["input_ids"].numel()
    assert batch["input_ids"].numel() == T and batch["cu_seqlens"].tolist() == [0, a["input_ids"].numel(), T]
    assert batch["labels"][a["input_ids"].numel() - 1] == -100            # no target crosses the sample boundary
    assert int((batch["labels"] != -100).sum()) == len("a chart") + 1 + len("hi there") + 1
    out = model(batch)
    loss = out[0] / out[1] if isinstance(out, tuple) else out
    assert torch.isfinite(loss)
    loss.backward()
    assert model.tile_format.image_newline.grad.abs().sum() > 0


def test_trainer_runs_the_tiled_recipe(tmp_path, capsys):
    import json
    import os
    from PIL import Image
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    Image.new("RGB", (120, 50), (10, 200, 30)).save(tmp_path / "a.png")
    recs = [{"messages": [{"role": "user", "content": "<image>\nwhat is this?"}, {"role": "assistant", "content": "a green card"}],
             "images": ["a.png"]}] * 4
    (tmp_path / "d.json").write_text(json.dumps(recs))
    args = load_config(os.path.join(root, "examples/deepseekvl2/tiny_native.yaml"),
                       [f"data.dataset_param.basic_parameters.dataset={tmp_path}/d.json",
                        f"data.dataset_param.basic_parameters.dataset_dir={tmp_path}", "training.train_iters=2"], world_size=1)
    hist = Trainer(args, device="cpu").train()
    assert len(hist) == 2 and all(h["loss"] == h["loss"] for h in hist)
    # the shipped text-only demo file runs as well
    args = load_config(os.path.join(root, "examples/deepseekvl2/tiny_native.yaml"),
                       [f"data.dataset_param.basic_parameters.dataset={root}/examples/deepseekvl2/demo.json", "training.train_iters=1"],
                       world_size=1)
    assert len(Trainer(args, device="cpu").train()) == 1
