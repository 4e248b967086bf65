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


def test_pretrain_vlm_reads_a_sharegpt_json_with_the_reference_data_schema(tmp_path, capsys):
    """``--mm-data`` in the reference's schema (examples/qwen2.5vl/data_7b.json) naming a real sharegpt file with images:
    the conversations go through the chat template + image processor, ``dynamic_batching`` packs them to the sequence
    length, and a resumed run continues after the samples already consumed."""
    from PIL import Image
    from mindspeed_mm_b200.runtime.legacy_entry import datasets_provider, pretrain
    img_dir = tmp_path / "images"
    img_dir.mkdir()
    recs = []
    for i in range(6):
        Image.new("RGB", (56 + 28 * (i % 2), 56), (40 * i, 10, 200 - 30 * i)).save(img_dir / f"{i}.png")
        recs.append({"messages": [{"role": "user", "content": f"<image>what is picture {i}?"},
                                  {"role": "assistant", "content": f"picture number {i} " * (1 + i)}],
                     "images": [f"images/{i}.png"]})
    (tmp_path / "sft.json").write_text(json.dumps(recs))
    data = {"dataset_param": {"dataset_type": "huggingface",
                              "preprocess_parameters": {"model_name_or_path": "./missing", "image_max_pixels": 12544,
                                                        "image_min_pixels": 0},
                              "basic_parameters": {"template": "qwen2vl", "dataset_dir": str(tmp_path), "dataset": "sft.json",
                                                   "cutoff_len": 256},
                              "attr": {"images": "images", "messages": "messages", "role_tag": "role",
                                       "content_tag": "content", "user_tag": "user", "assistant_tag": "assistant"}},
            "dataloader_param": {"dataloader_mode": "dynamic_batching", "drop_last": True, "shuffle": False,
                                 "sampler_type": "BaseRandomBatchSampler", "dynamic_batch_buffer_size": 3,
                                 "collate_param": {"model_name": "qwen2vl", "ignore_pad_token_for_loss": True}}}
    d = tmp_path / "data.json"
    d.write_text(json.dumps(data))
    argv = ["--mm-model", os.path.join(ROOT, "examples/qwen2.5vl/model_tiny.json"), "--mm-data", str(d), "--train-iters", "2",
            "--micro-batch-size", "1", "--global-batch-size", "1", "--lr", "1e-4", "--seq-length", "256", "--seed", "3"]
    hist = pretrain("vlm", argv, device="cpu")
    out = capsys.readouterr().out
    assert len(hist) == 2 and all(h["loss"] == h["loss"] for h in hist)
    assert "MultimodalConversationDataset with 6 samples" in out
    _reset()
    # packing: several conversations per micro-batch, never longer than the sequence length; resume skips consumed samples
    from mindspeed_mm_b200.config.legacy import parse_legacy_args
    from mindspeed_mm_b200.parallel.state import init_parallel_state
    from mindspeed_mm_b200.runtime.legacy_entry import model_provider
    args = parse_legacy_args(argv)
    ps = init_parallel_state(world_size=1, device_type="cpu")
    model = model_provider("vlm", args)
    first = next(datasets_provider("vlm", args, model, ps))
    assert first["cu_seqlens"].numel() > 2 and int(first["cu_seqlens"][-1]) <= 256 and "pixel_values" in first
    resumed = next(datasets_provider("vlm", args, model, ps, consumed_samples=3))
    assert resumed["input_ids"].shape != first["input_ids"].shape or not torch.equal(resumed["input_ids"], first["input_ids"])
    _reset()


def test_pretrain_sora_dreambooth_lora_with_prior_preservation(tmp_path):
    """DreamBooth-style subject fine-tuning through the generative entry point: images of a folder with an instance prompt,
    class images for the prior term, raw pixels encoded by the frozen VAE / text encoder, LoRA adapters on the
    predictor's attention projections as the only trainable parameters."""
    import numpy as np
    from PIL import Image
    from mindspeed_mm_b200.runtime.legacy_entry import pretrain
    rng = np.random.default_rng(0)
    inst, cls = tmp_path / "dog", tmp_path / "class"
    inst.mkdir()
    cls.mkdir()
    for d, n in ((inst, 4), (cls, 2)):
        for i in range(n):
            Image.fromarray(rng.integers(0, 255, (40, 48, 3), dtype=np.uint8)).save(d / f"{i}.png")
    model = {
        "load_video_features": False, "load_text_features": False, "task": "t2v",
        "diffusion": {"model_id": "wan_flow_match_scheduler", "num_train_timesteps": 1000, "shift": 5, "sigma_min": 0.0,
                      "extra_one_step": True},
        "predictor": {"model_id": "wandit", "dtype": "bf16", "model_type": "t2v", "patch_size": [1, 2, 2], "text_len": 16,
                      "in_dim": 4, "hidden_size": 64, "ffn_dim": 128, "freq_dim": 32, "text_dim": 32, "out_dim": 4,
                      "num_heads": 4, "num_layers": 2, "qk_norm": True, "cross_attn_norm": True, "eps": 1e-6},
        "ae": {"model_id": "wan_video_vae", "base_dim": 8, "z_dim": 4, "dim_mult": [1, 2, 2, 2], "num_res_blocks": 1,
               "latents_mean": [0] * 4, "latents_std": [1] * 4},
        "text_encoder": {"model_id": "UMT5", "vocab_size": 300, "d_model": 32, "d_kv": 8, "d_ff": 64, "num_layers": 1, "num_heads": 4},
        "lora": {"enable": True, "rank": 4, "alpha": 8, "target_modules": ["self_attn.qkv", "self_attn.proj_out", "cross_attn.proj_q"]},
        "prior_loss_weight": 0.5,
    }
    data = {"dataset_param": {"dataset_type": "dreambooth",
                              "basic_parameters": {"instance_data_dir": str(inst), "instance_prompt": "a photo of sks dog",
                                                   "class_data_dir": str(cls), "class_prompt": "a photo of a dog"},
                              "preprocess_parameters": {"resolution": 32, "text_len": 16}},
            "dataloader_param": {"dataloader_mode": "sampler", "shuffle": False, "drop_last": True, "pin_memory": False, "num_workers": 0}}
    m, d = tmp_path / "model.json", tmp_path / "data.json"
    m.write_text(json.dumps(model))
    d.write_text(json.dumps(data))
    hist = pretrain("sora", ["--mm-model", str(m), "--mm-data", str(d), "--train-iters", "3", "--micro-batch-size", "2",
                             "--global-batch-size", "2", "--lr", "1e-3"], device="cpu")
    assert len(hist) == 3 and all(torch.isfinite(torch.tensor(h["loss"])) for h in hist)
    _reset()
