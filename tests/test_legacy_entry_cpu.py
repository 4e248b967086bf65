"""Megatron-style entry points end to end on CPU: model JSON -> engine -> two steps; the FSDP2 sharding YAML is read."""
import json
import os

import torch

from mindspeed_mm_b200.config.legacy import load_fsdp2_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reset():
    from mindspeed_mm_b200.parallel.state import reset_parallel_state
    reset_parallel_state()


def test_fsdp2_yaml_is_normalised(tmp_path):
    y = tmp_path / "fsdp2.yaml"
    y.write_text("sharding_size: auto\nsub_modules_to_wrap:\n  - model.layers.{*}\nparam_dtype: bf16\nreduce_dtype: fp32\n"
                 "reshard_after_forward: true\nrecompute_modules:\n  - model.layers.{*}\nsome_new_key: 1\n")
    c = load_fsdp2_config(str(y))
    assert c["sharding_size"] is None and c["param_dtype"] is torch.bfloat16 and c["reduce_dtype"] is torch.float32
    assert c["sub_modules_to_wrap"] == ["model.layers.{*}"] and c["unknown_keys"] == ["some_new_key"]
    y.write_text("sharding_size: 4\n")
    assert load_fsdp2_config(str(y))["sharding_size"] == 4


def test_pretrain_vlm_and_sora_run_from_their_json(tmp_path, capsys):
    from mindspeed_mm_b200.runtime.legacy_entry import pretrain
    y = tmp_path / "fsdp2.yaml"
    y.write_text("sharding_size: 8\nparam_dtype: bf16\nreduce_dtype: fp32\nodd_key: true\n")
    hist = pretrain("vlm", ["--mm-model", os.path.join(ROOT, "examples/qwen2.5vl/model_tiny.json"), "--train-iters", "2",
                            "--micro-batch-size", "1", "--global-batch-size", "1", "--lr", "1e-4", "--seq-length", "256",
                            "--use-torch-fsdp2", "--fsdp2-config-path", str(y), "--log-tps", "--seed", "3"], device="cpu")
    out = capsys.readouterr().out
    assert len(hist) == 2 and all(h["loss"] == h["loss"] for h in hist)
    assert "sharding_size=8" in out and "odd_key" in out and "iteration        2/       2" in out
    _reset()
    tiny = json.load(open(os.path.join(ROOT, "examples/sdxl/pretrain_model_tiny.json")))
    m = tmp_path / "sdxl.json"
    m.write_text(json.dumps(tiny))
    d = tmp_path / "data.json"
    d.write_text(json.dumps({"dataset_param": {"basic_parameters": {"frames": 1, "height": 8, "width": 8, "text_len": 5}}}))
    hist = pretrain("sora", ["--mm-model", str(m), "--mm-data", str(d), "--train-iters", "2", "--micro-batch-size", "2",
                             "--global-batch-size", "2", "--lr", "1e-4"], device="cpu")
    assert len(hist) == 2 and all(torch.isfinite(torch.tensor(h["loss"])) for h in hist)
    _reset()
