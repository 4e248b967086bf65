"""File-backed multimodal dataset: processor parity with transformers, template label masking, collation."""
import json
import os

import numpy as np
import pytest
import torch

from mindspeed_mm_b200.data.multimodal import (ByteTokenizer, ChatTemplate, FeatureDataset, MultimodalConversationDataset,
                                               Qwen2VLImageProcessor, smart_resize)


def test_smart_resize_budget_and_divisibility():
    for h, w in [(111, 203), (3000, 4000), (20, 20), (28, 2800)]:
        rh, rw = smart_resize(h, w, 28, 56 * 56, 28 * 28 * 1280)
        assert rh % 28 == 0 and rw % 28 == 0 and 56 * 56 <= rh * rw <= 28 * 28 * 1280


def test_image_processor_matches_transformers():
    PIL = pytest.importorskip("PIL.Image")
    from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor as HP
    rng = np.random.default_rng(0)
    img = PIL.fromarray((rng.random((111, 203, 3)) * 255).astype("uint8"))
    want = HP(min_pixels=56 * 56, max_pixels=28 * 28 * 1280)(images=[img], return_tensors="pt")
    rows, grid = Qwen2VLImageProcessor(max_pixels=28 * 28 * 1280)(img)
    assert tuple(want["image_grid_thw"][0].tolist()) == grid
    assert (want["pixel_values"] - rows).abs().max() < 0.02      # one uint8 step after normalisation


def test_conversation_dataset_masks_everything_but_assistant(tmp_path):
    PIL = pytest.importorskip("PIL.Image")
    PIL.fromarray(np.zeros((60, 90, 3), dtype="uint8")).save(tmp_path / "a.png")
    recs = [{"messages": [{"role": "user", "content": "<image>What is this?"}, {"role": "assistant", "content": "A test."}],
             "images": ["a.png"]},
            {"conversations": [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "hello"}]},
            {"messages": [{"role": "user", "content": "no marker"}, {"role": "assistant", "content": "ok"}], "images": ["a.png"]}]
    (tmp_path / "d.json").write_text(json.dumps(recs))
    ds = MultimodalConversationDataset(files=["d.json"], dataset_dir=str(tmp_path), cutoff_len=512)
    tok = ByteTokenizer()
    s = ds[0]
    n_img = int(s["image_grid_thw"].prod(-1).sum()) // 4
    assert (s["input_ids"] == tok.special_ids["<|image_pad|>"]).sum() == n_img
    assert tok.decode(s["input_ids"][s["labels"] != -100].tolist()) == "A test.<|im_end|>"
    assert ds[1]["pixel_values"].shape[0] == 0
    s2 = ds[2]                                             # marker added in front of the first user turn
    assert (s2["input_ids"] == tok.special_ids["<|image_pad|>"]).sum() == s2["pixel_values"].shape[0] // 4
    # a cut-off inside the placeholders drops the image instead of leaving a partial run
    short = MultimodalConversationDataset(files=["d.json"], dataset_dir=str(tmp_path), cutoff_len=48)[0]
    assert (short["input_ids"] == tok.special_ids["<|image_pad|>"]).sum() == 0 and short["pixel_values"].shape[0] == 0


def test_samples_flow_through_packed_collator(tmp_path):
    PIL = pytest.importorskip("PIL.Image")
    from mindspeed_mm_b200.data.collate import PackedVLMCollator
    PIL.fromarray(np.zeros((56, 56, 3), dtype="uint8")).save(tmp_path / "a.png")
    recs = [{"messages": [{"role": "user", "content": "<image>x"}, {"role": "assistant", "content": "y"}], "images": ["a.png"]}] * 2
    (tmp_path / "d.jsonl").write_text("\n".join(json.dumps(r) for r in recs))
    ds = MultimodalConversationDataset(files=["d.jsonl"], dataset_dir=str(tmp_path))
    tok = ByteTokenizer()
    coll = PackedVLMCollator(tok.special_ids["<|image_pad|>"], tok.special_ids["<|vision_start|>"])
    batch = coll([ds[0], ds[1]])
    assert batch["input_ids"].shape[0] == 2 * ds[0]["input_ids"].shape[0]
    assert batch["pixel_values"].shape[0] == 2 * ds[0]["pixel_values"].shape[0]


def test_feature_dataset(tmp_path):
    for i in range(3):
        torch.save({"latents": torch.randn(4, 3, 8, 8), "prompt": torch.randn(5, 16)}, tmp_path / f"{i}.pt")
    (tmp_path / "index.txt").write_text("\n".join(f"{i}.pt" for i in range(3)))
    ds = FeatureDataset(index=str(tmp_path / "index.txt"), data_folder=str(tmp_path))
    assert len(ds) == 3 and ds[1]["latents"].shape == (4, 3, 8, 8) and ds[1]["prompt_mask"].all()


def test_dreambooth_dataset_instance_and_class_images(tmp_path):
    import numpy as np
    import pytest
    from PIL import Image
    from mindspeed_mm_b200.data.multimodal import DreamBoothDataset
    from mindspeed_mm_b200.models.registry import data_register
    rng = np.random.default_rng(0)
    inst, cls = tmp_path / "dog", tmp_path / "class"
    inst.mkdir()
    cls.mkdir()
    for d, n in ((inst, 3), (cls, 2)):
        for i in range(n):
            Image.fromarray(rng.integers(0, 255, (40 + 8 * i, 56, 3), dtype=np.uint8)).save(d / f"{i}.png")
    (inst / "notes.txt").write_text("ignored")
    ds = DreamBoothDataset(instance_data_dir=str(inst), instance_prompt="a photo of sks dog", class_data_dir=str(cls),
                           class_prompt="a photo of a dog", repeats=2, height=32, width=32, text_len=24)
    assert len(ds) == 6 and data_register.get("dreambooth") is DreamBoothDataset
    it = ds[4]
    assert it["video"].shape == (3, 1, 32, 32) and it["class_video"].shape == (3, 1, 32, 32)
    assert float(it["video"].min()) >= -1.0 and float(it["video"].max()) <= 1.0
    assert int(it["prompt_mask"].sum()) == len("a photo of sks dog") and int(it["class_prompt_mask"].sum()) == len("a photo of a dog")
    plain = DreamBoothDataset(instance_data_dir=str(inst), instance_prompt="x", height=16, width=16, text_len=4)
    assert "class_video" not in plain[0] and len(plain) == 3
    with pytest.raises(ValueError):
        DreamBoothDataset(instance_data_dir=str(tmp_path / "missing"), instance_prompt="x")
