"""Config loaders: golden parses of the reference's own example files (when the tree is mounted) and of
this repo's examples."""
import glob
import json
import os

import pytest
import yaml

from mindspeed_mm_b200.config import (ConfigNode, MMConfig, load_config, module_name_match, parse_legacy_args,
                                      yaml_to_argv)
from mindspeed_mm_b200.config.security import check_path
from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig

# the reference's recipe folder: next to this repository unless MM_REFERENCE_EXAMPLES points elsewhere
REF = os.environ.get("MM_REFERENCE_EXAMPLES") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "examples")
HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_config_node_roundtrip():
    d = {"a": 1, "b": {"c": [1, 2], "dtype": "bf16"}}
    n = ConfigNode(d)
    import torch
    assert n.b.dtype == torch.bfloat16 and n.b.c == [1, 2] and n.get("zz", 5) == 5
    assert n.update_unuse(a=3, q=4) == {"q": 4} and n.a == 3


def test_legacy_cli_and_json(tmp_path):
    m = tmp_path / "model.json"
    m.write_text(json.dumps({"model_id": "qwen2_5vl", "text_decoder": {"num_layers": 2}}))
    args = parse_legacy_args(["--tensor-model-parallel-size", "2", "--bf16", "--lr", "1e-5", "--mm-model", str(m),
                              "--some-unknown-flag", "7", "--other-flag", "--log-tps"])
    assert args.tensor_model_parallel_size == 2 and args.bf16 and args.lr == 1e-5 and args.log_tps
    assert args.some_unknown_flag == "7" and args.other_flag is True
    assert args.mm.model.text_decoder.num_layers == 2


def test_megatron_yaml_flatten(tmp_path):
    y = tmp_path / "c.yaml"
    y.write_text(yaml.safe_dump({"gpt_args": {"train": {"micro_batch_size": 2, "bf16": True, "use_x": False},
                                              "lr": 1e-5, "list_arg": [1, 2]},
                                 "MM_TOOL_PATH": "tools.json", "model": {"model_id": "x"}, "data": {"a": 1}}))
    argv = yaml_to_argv(str(y))
    i = argv.index("--micro-batch-size")
    assert argv[i + 1] == "2" and "--bf16" in argv and "--use-x" not in argv
    assert argv.count("--list-arg") == 2 and argv[-1] == "tools.json"


def test_native_yaml_and_overrides(tmp_path):
    y = tmp_path / "n.yaml"
    y.write_text(yaml.safe_dump({
        "parallel": {"fully_shard_parallel_size": "auto", "ulysses_parallel_size": 2,
                     "fsdp_plan": {"apply_modules": ["model.layers.{*}"], "num_to_forward_prefetch": 1}},
        "model": {"model_id": "qwen2_5vl", "custom_key": 3},
        "training": {"lr": 1e-4, "micro_batch_size": 2, "gradient_accumulation_steps": 2, "plugin": ["a", "b"]},
        "features": {"recompute": True, "loss_cfg": {"loss_type": "per_token_loss"}}}))
    a = load_config(str(y), ["training.lr=3e-4", "training.plugin.1=zz", "tools.profile.enable=true"], world_size=8)
    assert a.training.lr == 3e-4 and a.training.plugin == ["a", "zz"] and a.tools.profile.enable
    assert a.parallel.fully_shard_parallel_size == 8 and a.parallel.data_parallel_size == 4
    assert a.training.global_batch_size == 2 * 2 * 4 and a.model.custom_key == 3
    assert a.features.loss_cfg.loss_type == "per_token_loss"
    with pytest.raises(ValueError):
        load_config(str(y), ["parallel.ulysses_parallel_size=3"], world_size=8)


def test_module_name_match():
    assert module_name_match("model.layers.{*}", "model.layers.12")
    assert not module_name_match("model.layers.{*}", "model.layers.12.mlp")
    assert module_name_match("model.layers.{0-3,7}.mlp", "model.layers.7.mlp")
    assert not module_name_match("model.layers.{0-3,7}.mlp", "model.layers.5.mlp")


def test_path_checker(tmp_path):
    f = tmp_path / "x.json"
    f.write_text("{}")
    link = tmp_path / "l.json"
    os.symlink(f, link)
    assert check_path(str(f), "p", base_dir=str(tmp_path), warn=lambda *_: None)
    assert not check_path(str(link), "p", base_dir=str(tmp_path), warn=lambda *_: None)
    assert not check_path(str(f), "p", base_dir=str(tmp_path / "sub"), warn=lambda *_: None)


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference examples not mounted")
def test_reference_examples_parse():
    # every model/data JSON of the reference loads into a tree; the VLM ones build a model config
    n = 0
    for p in glob.glob(os.path.join(REF, "qwen2.5vl", "model_*.json")):
        cfg = MMConfig({"model": p}).model
        q = Qwen25VLConfig.from_mm_json(cfg.to_dict())
        assert q.text.hidden_size % q.text.num_attention_heads == 0
        n += 1
    assert n >= 3
    m7 = Qwen25VLConfig.from_mm_json(json.load(open(os.path.join(REF, "qwen2.5vl", "model_7b.json"))))
    assert (m7.text.num_layers, m7.text.hidden_size, m7.text.num_key_value_heads, m7.vision.depth) == (28, 3584, 4, 32)
    for p in glob.glob(os.path.join(REF, "*", "*config*.yaml")):
        try:
            doc = yaml.safe_load(open(p))
        except yaml.YAMLError:          # one reference recipe defines a YAML anchor twice
            continue
        if isinstance(doc, dict) and "parallel" in doc and "training" in doc:
            a = load_config(p, world_size=8)
            assert a.training.micro_batch_size >= 1
            n += 1
    assert n >= 5


def test_validate_args_reports_inconsistent_flags_and_derives_sizes():
    import pytest
    from mindspeed_mm_b200.config.legacy import parse_legacy_args, validate_args
    ok = parse_legacy_args(["--tensor-model-parallel-size", "2", "--pipeline-model-parallel-size", "2", "--context-parallel-size", "2",
                            "--context-parallel-algo", "hybrid_cp_algo", "--ulysses-degree-in-cp", "2", "--micro-batch-size", "1",
                            "--global-batch-size", "8", "--seq-length", "4096", "--num-layers", "8", "--num-attention-heads", "16",
                            "--sequence-parallel", "--bf16"], check_paths=False)
    d = validate_args(ok, world_size=16)
    assert (d.data_parallel_size, d.num_micro_batches, d.ulysses_size, d.ring_size, d.sequence_parallel, d.params_dtype) == (
        2, 4, 2, 1, True, "bf16")
    # tensor parallel 1 switches sequence parallelism off, as Megatron does
    assert validate_args(parse_legacy_args(["--sequence-parallel"], check_paths=False), 4).sequence_parallel is False
    bad = parse_legacy_args(["--tensor-model-parallel-size", "4", "--bf16", "--fp16", "--micro-batch-size", "2", "--global-batch-size",
                             "6", "--min-lr", "1e-3", "--lr", "1e-4", "--num-layers", "6", "--pipeline-model-parallel-size", "1",
                             "--recompute-method", "block", "--use-torch-fsdp2"], check_paths=False)
    with pytest.raises(ValueError) as e:
        validate_args(bad, world_size=8)
    msg = str(e.value)
    for frag in ("--global-batch-size 6", "--bf16 and --fp16", "--min-lr", "--recompute-method needs", "--use-torch-fsdp2 shards"):
        assert frag in msg, (frag, msg)
    with pytest.raises(ValueError, match="not divisible by tensor"):
        validate_args(parse_legacy_args(["--tensor-model-parallel-size", "3"], check_paths=False), 8)
    ring = parse_legacy_args(["--context-parallel-size", "4", "--context-parallel-algo", "megatron_cp_algo", "--seq-length", "1028"],
                             check_paths=False)
    with pytest.raises(ValueError, match="zig-zag"):
        validate_args(ring, 4)
