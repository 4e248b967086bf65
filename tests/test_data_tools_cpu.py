"""Dataset preparation helpers: mock conversations load through the real dataset class; LLaVA records are re-laid."""
import json
import os

from mindspeed_mm_b200.data import data_tools as dt


def test_mock_dataset_is_readable_by_the_conversation_dataset(tmp_path):
    path = dt.write_mock_dataset(str(tmp_path), num_pics=2, text_length=200, num_samples=3, width=56, height=56)
    recs = json.load(open(path))
    assert len(recs) == 3 and recs[0]["images"] == ["test_pic_h56_w56.jpg"] * 2
    assert recs[0]["messages"][0]["content"].count("<image>") == 2
    assert os.path.exists(tmp_path / "test_pic_h56_w56.jpg")
    from mindspeed_mm_b200.data.multimodal import MultimodalConversationDataset
    ds = MultimodalConversationDataset(files=[path], dataset_dir=str(tmp_path), cutoff_len=4096)
    s = ds[0]
    assert len(ds) == 3 and s["input_ids"].numel() > 100 and s["image_grid_thw"].shape[0] == 2
    # the text budget follows the token counter
    longer = dt.write_mock_dataset(str(tmp_path / "b"), num_pics=1, text_length=200, num_samples=1, width=28, height=28,
                                   count_tokens=lambda s: 1)
    a, b = json.load(open(path))[0]["messages"][1]["content"], json.load(open(longer))[0]["messages"][1]["content"]
    assert len(b) > len(a)


def test_llava_records_are_converted_and_missing_pictures_skipped(tmp_path):
    (tmp_path / "train2017").mkdir()
    (tmp_path / "train2017" / "1.jpg").write_bytes(b"x")
    recs = [{"image": "1.jpg", "conversations": [{"from": "human", "value": "<image>\nwhat?"}, {"from": "gpt", "value": "a cat"}]},
            {"image": "2.jpg", "conversations": [{"from": "human", "value": "q"}, {"from": "gpt", "value": "a"}]},
            {"conversations": [{"from": "human", "value": "text only"}, {"from": "gpt", "value": "ok"}]}]
    out = dt.convert_llava_instruct(recs, str(tmp_path))
    assert len(out) == 2 and out[0]["images"] == [os.path.join("train2017", "1.jpg")] and out[1]["images"] == []
    assert out[0]["messages"] == [{"role": "user", "content": "<image>\nwhat?"}, {"role": "assistant", "content": "a cat"}]
    src = tmp_path / "in.json"
    src.write_text(json.dumps(recs))
    assert dt.main(["llava", "--llava-json", str(src), "--image-root", str(tmp_path), "--out", str(tmp_path / "o" / "out.json")]) == 0
    assert dt.main(["llava", "--llava-json", str(src), "--out", str(tmp_path / "o" / "out.json")]) == 1      # never overwrites
    try:
        dt.convert_llava_instruct([{"conversations": [{"from": "robot", "value": "x"}]}])
        raise AssertionError
    except ValueError:
        pass
