"""Checkpoint formats: operator algebra, HF <-> internal <-> Megatron round trips, resume, resharding,
and numerical parity of the model against HuggingFace's Qwen2.5-VL on a tiny config."""
import json
import os

import pytest
import torch

from mindspeed_mm_b200.api import stable_init_fn
from mindspeed_mm_b200.checkpoint import hf as hfio
from mindspeed_mm_b200.checkpoint import megatron as mm
from mindspeed_mm_b200.checkpoint.convert_cli import main as mm_convert
from mindspeed_mm_b200.checkpoint.operators import (ExpertStack, QKVMerge, concat_to_interleaved,
                                                    interleaved_to_concat, merge_glu, split_glu)
from mindspeed_mm_b200.checkpoint.sharded import DistributedCheckpointer
from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig


def small_cfg():
    cfg = Qwen25VLConfig.tiny()
    cfg.text.num_layers = 2
    cfg.vision.depth = 2
    cfg.vision.fullatt_block_indexes = (1,)
    cfg.vision.intermediate_size = 300      # not a multiple of 64 -> exercises the FFN pad
    return cfg


def fake_hf_state(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    t, v = cfg.text, cfg.vision
    sd = {}
    R = lambda *s: torch.randn(*s, generator=g) * 0.05
    sd["model.visual.patch_embed.proj.weight"] = R(v.hidden_size, 3, 2, 14, 14)
    for i in range(v.depth):
        p = f"model.visual.blocks.{i}."
        sd[p + "norm1.weight"], sd[p + "norm2.weight"] = 1 + R(v.hidden_size), 1 + R(v.hidden_size)
        sd[p + "attn.qkv.weight"], sd[p + "attn.qkv.bias"] = R(3 * v.hidden_size, v.hidden_size), R(3 * v.hidden_size)
        sd[p + "attn.proj.weight"], sd[p + "attn.proj.bias"] = R(v.hidden_size, v.hidden_size), R(v.hidden_size)
        for n in ("gate_proj", "up_proj"):
            sd[p + f"mlp.{n}.weight"], sd[p + f"mlp.{n}.bias"] = R(v.intermediate_size, v.hidden_size), R(v.intermediate_size)
        sd[p + "mlp.down_proj.weight"], sd[p + "mlp.down_proj.bias"] = R(v.hidden_size, v.intermediate_size), R(v.hidden_size)
    m = v.hidden_size * 4
    sd["model.visual.merger.ln_q.weight"] = 1 + R(v.hidden_size)
    sd["model.visual.merger.mlp.0.weight"], sd["model.visual.merger.mlp.0.bias"] = R(m, m), R(m)
    sd["model.visual.merger.mlp.2.weight"], sd["model.visual.merger.mlp.2.bias"] = R(v.out_hidden_size, m), R(v.out_hidden_size)
    sd["model.language_model.embed_tokens.weight"] = R(t.vocab_size, t.hidden_size)
    for i in range(t.num_layers):
        p = f"model.language_model.layers.{i}."
        for n, rows in (("q", t.num_attention_heads), ("k", t.num_key_value_heads), ("v", t.num_key_value_heads)):
            sd[p + f"self_attn.{n}_proj.weight"] = R(rows * t.head_dim, t.hidden_size)
            sd[p + f"self_attn.{n}_proj.bias"] = R(rows * t.head_dim)
        sd[p + "self_attn.o_proj.weight"] = R(t.hidden_size, t.hidden_size)
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = R(t.intermediate_size, t.hidden_size), R(t.intermediate_size, t.hidden_size)
        sd[p + "mlp.down_proj.weight"] = R(t.hidden_size, t.intermediate_size)
        sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = 1 + R(t.hidden_size), 1 + R(t.hidden_size)
    sd["model.language_model.norm.weight"] = 1 + R(t.hidden_size)
    sd["lm_head.weight"] = R(t.vocab_size, t.hidden_size)
    return sd


def test_qkv_interleave_roundtrip():
    q, k, v = torch.arange(8.).view(8, 1), 100 + torch.arange(4.).view(4, 1), 200 + torch.arange(4.).view(4, 1)
    cat = torch.cat([q, k, v])
    inter = concat_to_interleaved(cat, 2, [8, 4, 4])
    assert inter.flatten().tolist() == [0, 1, 2, 3, 100, 101, 200, 201, 4, 5, 6, 7, 102, 103, 202, 203]
    assert torch.equal(interleaved_to_concat(inter, 2, [4, 2, 2]), cat)


def test_glu_split_merge():
    t = torch.arange(16.).view(8, 2)
    parts = split_glu(t, 2)
    assert torch.equal(parts[0], torch.cat([t[0:2], t[4:6]]))
    assert torch.equal(merge_glu(parts), t)


def test_expert_stack():
    sd = {f"l.0.experts.{e}.w": torch.full((2, 3), float(e)) for e in range(4)}
    op = ExpertStack("l.{i}.experts.{e}.w", "l.{i}.experts.w_stacked")
    op.apply(sd)
    assert sd["l.0.experts.w_stacked"].shape == (4, 3, 2)
    op.revert(sd)
    assert torch.equal(sd["l.0.experts.2.w"], torch.full((2, 3), 2.0))


def test_hf_internal_roundtrip_and_model_load():
    cfg = small_cfg()
    hf_sd = fake_hf_state(cfg)
    ops = hfio.qwen25vl_ops(cfg)
    internal = hfio.to_internal(hf_sd, ops)
    with torch.device("meta"):
        model = Qwen25VLModel(cfg)
    names = {n: p.shape for n, p in model.named_parameters()}
    assert set(names) == set(internal), (set(names) ^ set(internal))
    for n, s in names.items():
        assert tuple(internal[n].shape) == tuple(s), n
    back = hfio.to_hf(internal, hfio.qwen25vl_ops(cfg))
    assert set(back) == set(hf_sd)
    for k in hf_sd:
        assert torch.equal(back[k], hf_sd[k]), k


def test_hf_mm_roundtrip_tp_pp(tmp_path):
    cfg = small_cfg()
    t, v = cfg.text, cfg.vision
    hf_sd = fake_hf_state(cfg)
    mk = lambda: mm.qwen25vl_mm_ops(t.num_attention_heads, t.num_key_value_heads, t.head_dim, v.num_heads)
    stages = mm.hf_to_mm(hf_sd, mk(), tp=2, vit_layers=[2, 0], llm_layers=[1, 1])
    assert len(stages) == 2 and len(stages[0]) == 2
    s0, s1 = stages[0][0], stages[1][0]
    assert "text_decoder.embedding.word_embeddings.weight" in s0 and "text_decoder.output_layer.weight" in s1
    assert "text_decoder.decoder.layers.0.mlp.linear_fc1.weight" in s1          # renumbered from global layer 1
    assert not any(k.startswith("image_encoder") for k in s1)
    assert s0["text_decoder.decoder.layers.0.self_attention.linear_qkv.weight"].shape[0] == \
        (t.num_attention_heads + 2 * t.num_key_value_heads) * t.head_dim // 2
    mm.save_mm(stages, str(tmp_path / "mm"))
    assert os.path.exists(tmp_path / "mm" / "release" / "mp_rank_01_001" / "model_optim_rng.pt")
    assert open(tmp_path / "mm" / "latest_checkpointed_iteration.txt").read() == "release"
    back = mm.mm_to_hf(mm.load_mm(str(tmp_path / "mm")), mk(), [2, 0], [1, 1])
    assert set(back) == set(hf_sd)
    for k in hf_sd:
        assert torch.equal(back[k], hf_sd[k]), k


def test_mm_convert_cli(tmp_path):
    cfg = small_cfg()
    t, v = cfg.text, cfg.vision
    hf_dir = tmp_path / "hf"
    hfio.save_sharded(fake_hf_state(cfg), str(hf_dir), max_shard_bytes=20 << 20)
    assert os.path.exists(hf_dir / hfio.INDEX)
    json.dump({"text_config": {"num_attention_heads": t.num_attention_heads, "num_key_value_heads": t.num_key_value_heads,
                               "hidden_size": t.hidden_size, "num_hidden_layers": t.num_layers},
               "vision_config": {"num_heads": v.num_heads, "depth": v.depth}}, open(hf_dir / "config.json", "w"))
    assert mm_convert(["Qwen2_5_VLConverter", "hf_to_mm", "--cfg.mm_dir", str(tmp_path / "mm"), "--cfg.hf_config.hf_dir",
                       str(hf_dir), "--cfg.parallel_config.llm_pp_layers", "[[1,1]]",
                       "--cfg.parallel_config.vit_pp_layers", "[[2,0]]", "--cfg.parallel_config.tp_size", "2"]) == 0
    assert mm_convert(["Qwen2_5_VLConverter", "resplit", "--cfg.source_dir", str(tmp_path / "mm"), "--cfg.target_dir",
                       str(tmp_path / "mm2"), "--cfg.hf_config.hf_dir", str(hf_dir),
                       "--cfg.source_parallel_config.llm_pp_layers", "[[1,1]]", "--cfg.source_parallel_config.vit_pp_layers",
                       "[[2,0]]", "--cfg.source_parallel_config.tp_size", "2", "--cfg.target_parallel_config.llm_pp_layers",
                       "[[2]]", "--cfg.target_parallel_config.vit_pp_layers", "[[2]]",
                       "--cfg.target_parallel_config.tp_size", "1"]) == 0
    assert mm_convert(["Qwen2_5_VLConverter", "mm_to_hf", "--cfg.save_hf_dir", str(tmp_path / "hf2"), "--cfg.mm_dir",
                       str(tmp_path / "mm2"), "--cfg.hf_config.hf_dir", str(hf_dir)]) == 0
    a, b = hfio.load_state_dict(str(hf_dir)), hfio.load_state_dict(str(tmp_path / "hf2"))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    assert mm_convert(["Qwen2_5_VLConverter", "hf_to_dcp", "--cfg.hf_dir", str(hf_dir), "--cfg.dcp_dir", str(tmp_path / "dcp")]) == 0
    assert mm_convert(["Qwen2_5_VLConverter", "dcp_to_hf", "--cfg.hf_dir", str(hf_dir), "--cfg.dcp_dir", str(tmp_path / "dcp"),
                       "--cfg.save_hf_dir", str(tmp_path / "hf3")]) == 0
    c = hfio.load_state_dict(str(tmp_path / "hf3"))
    assert set(a) == set(c) and all(torch.equal(a[k], c[k]) for k in a)


def _engine(cfg, world_rank=(1, 0)):
    with torch.device("meta"):
        model = Qwen25VLModel(cfg)
    eng = FSDPEngine(model.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=1e-3))
    eng.materialize(stable_init_fn(0.02, 0))
    return model, eng


def test_engine_hf_save_load_and_sharded_resume(tmp_path):
    from bench import make_batches
    cfg = small_cfg()
    cfg.vision.intermediate_size = 320
    model, eng = _engine(cfg)
    batch = make_batches(cfg, 1, 512, 1, 1, 224, 0, pin=False)[0]

    def step(m, e):
        e.set_lr(1e-3)
        ls, n = m(batch, run=e.run)
        (ls / n).backward()
        e.end_micro_step()
        e.finish_step()
        return float((ls / n).detach())

    step(model, eng)
    ck = DistributedCheckpointer(str(tmp_path / "ck"))
    ck.save(1, eng, {"iteration": 1})
    hfio.save_engine_as_hf(eng, str(tmp_path / "hf"), hfio.qwen25vl_ops(cfg))
    l2 = step(model, eng)
    # resume from the sharded checkpoint: same next loss
    model2, eng2 = _engine(cfg)
    extra = DistributedCheckpointer(str(tmp_path / "ck")).load(eng2)
    assert extra["iteration"] == 1
    assert abs(step(model2, eng2) - l2) < 1e-5
    # weights-only load from the HF export reproduces the same forward loss
    model3, eng3 = _engine(cfg)
    assert hfio.load_hf_into_engine(eng3, str(tmp_path / "hf"), hfio.qwen25vl_ops(cfg)) == []
    with torch.no_grad():
        ls, n = model3(batch, run=eng3.run)
    assert abs(float(ls / n) - l2) < 1e-4


def test_parity_with_transformers_tiny():
    tr = pytest.importorskip("transformers")
    try:
        from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    except Exception:  # noqa: BLE001
        pytest.skip("transformers lacks Qwen2.5-VL")
    torch.manual_seed(1234)          # the HF twin is randomly initialised: make it independent of the test order
    cfg = small_cfg()
    cfg.vision.intermediate_size = 320
    t, v = cfg.text, cfg.vision
    text_cfg = dict(vocab_size=t.vocab_size, hidden_size=t.hidden_size, intermediate_size=t.intermediate_size,
                    num_hidden_layers=t.num_layers, num_attention_heads=t.num_attention_heads,
                    num_key_value_heads=t.num_key_value_heads, rms_norm_eps=t.rms_norm_eps, rope_theta=t.rope_theta,
                    rope_scaling={"type": "mrope", "mrope_section": list(t.mrope_section), "rope_type": "default"},
                    max_position_embeddings=4096, tie_word_embeddings=False)
    vis_cfg = dict(depth=v.depth, hidden_size=v.hidden_size, intermediate_size=v.intermediate_size, num_heads=v.num_heads,
                   out_hidden_size=v.out_hidden_size, patch_size=14, spatial_merge_size=2, temporal_patch_size=2,
                   window_size=112, fullatt_block_indexes=list(v.fullatt_block_indexes), in_channels=3)
    try:
        hcfg = Qwen2_5_VLConfig(text_config=text_cfg, vision_config=vis_cfg, image_token_id=cfg.image_token_id,
                                video_token_id=cfg.video_token_id, vision_start_token_id=cfg.vision_start_token_id)
        hcfg._attn_implementation = "eager"
        hf = Qwen2_5_VLForConditionalGeneration(hcfg).float().eval()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"cannot build HF tiny model on this transformers version: {e}")
    hf_sd = {k: v_.detach().clone() for k, v_ in hf.state_dict().items()}
    with torch.device("meta"):
        model = Qwen25VLModel(cfg)
    eng = FSDPEngine(model.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32)
    eng.materialize(stable_init_fn(0.02, 0))
    internal = hfio.to_internal(hf_sd, hfio.qwen25vl_ops(cfg))
    missing = eng.load_full_params(lambda n, s: internal.get(n))
    assert missing == []
    from bench import make_batches
    batch = make_batches(cfg, 1, 384, 1, 1, 224, 0, pin=False)[0]
    with torch.no_grad():
        loss_sum, n = model(batch, run=eng.run)
        out = hf(input_ids=batch["input_ids"][None], pixel_values=batch["pixel_values"],
                 image_grid_thw=batch["image_grid_thw"], attention_mask=torch.ones(1, batch["n_tokens"], dtype=torch.long))
        logits = out.logits[0].float()
        ref = torch.nn.functional.cross_entropy(logits, batch["labels"], ignore_index=-100, reduction="sum")
    assert abs(float(loss_sum) - float(ref)) / float(ref) < 2e-4, (float(loss_sum), float(ref))


def test_torch_dcp_checkpoint_written_by_two_ranks_resumes_on_one(tmp_path):
    """DCP layout of the reference's native trainer: iter_XXXXXXX/ + extra_state/ + tracker, Hugging Face parameter
    names, row-sharded tensors.  Written by 2 gloo ranks (background save), resumed by 1 process: same next loss."""
    import re
    import subprocess
    import sys as _sys
    here = os.path.dirname(os.path.abspath(__file__))
    _sys.path.insert(0, here)
    import dist_dcp_check as dc
    from mindspeed_mm_b200.checkpoint.dcp import TorchDCPCheckpointer
    ck_dir = str(tmp_path / "dcp")
    cmd = [_sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 200), os.path.join(here, "dist_dcp_check.py"), ck_dir, "--async"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    want = float(re.search(r"next_loss=([\d.]+)", r.stdout).group(1))
    it = os.path.join(ck_dir, "iter_0000001")
    assert open(os.path.join(ck_dir, "latest_checkpointed_iteration.txt")).read() == "1"
    assert os.path.exists(os.path.join(it, ".metadata")) and os.path.exists(os.path.join(it, "extra_state", "extra_state_rank_1.pt"))
    from torch.distributed.checkpoint import FileSystemReader
    keys = set(FileSystemReader(it).read_metadata().state_dict_metadata)
    assert "model.model.language_model.layers.0.self_attn.q_proj.weight" in keys          # un-fused HF names
    assert "optimizer.state.model.language_model.layers.0.mlp.gate_proj.weight.exp_avg_sq" in keys
    cfg = dc.small_cfg()
    m, e = dc.build(cfg, False)
    extra = TorchDCPCheckpointer(ck_dir, ops=hfio.qwen25vl_ops(cfg)).load(e)
    assert extra["iteration"] == 1 and extra["consumed_train_samples"] == 2
    from bench import make_batches
    b = make_batches(cfg, 2, 300, 1, 1, 224, 0, pin=False)
    assert abs(dc.step(m, e, b[1]) - want) < 1e-5


def test_hf_to_dcp_release_checkpoint_loads_into_the_engine(tmp_path):
    """``mm-convert ... hf_to_dcp`` writes <dir>/release as DCP with HF names: the trainer-side checkpointer loads it
    (weights only, no optimizer / extra state)."""
    from mindspeed_mm_b200.checkpoint.convert_cli import Qwen2_5_VLConverter
    from mindspeed_mm_b200.checkpoint.dcp import TorchDCPCheckpointer
    import dist_dcp_check as dc
    cfg = dc.small_cfg()
    hf_dir, dcp_dir = str(tmp_path / "hf"), str(tmp_path / "dcp")
    sd = fake_hf_state(cfg)
    hfio.save_sharded(sd, hf_dir)
    Qwen2_5_VLConverter.hf_to_dcp({"hf_dir": hf_dir, "dcp_dir": dcp_dir})
    m, e = dc.build(cfg, False)
    assert TorchDCPCheckpointer(None, dcp_dir, ops=hfio.qwen25vl_ops(cfg)).load(e) == {}
    got = dict(e.named_full_params())
    want = hfio.to_internal({k: v.clone() for k, v in sd.items()}, hfio.qwen25vl_ops(cfg))
    for n, t in want.items():
        assert torch.allclose(got[n].float(), t.float(), atol=1e-6), n


def test_mm_convert_qwen3vl_dcp_and_expert_commands(tmp_path):
    """Qwen3VLConverter: hf_to_dcp stores the fused experts 2-D under the ``model.`` prefix and dcp_to_hf restores the
    Hugging Face files; moe_expert merges per-expert tensors into the fused pair and splits them again."""
    import json
    E, H, F = 4, 8, 6
    torch.manual_seed(0)
    hf = {"model.language_model.embed_tokens.weight": torch.randn(16, H), "lm_head.weight": torch.randn(16, H),
          "model.language_model.layers.0.mlp.experts.gate_up_proj": torch.randn(E, H, 2 * F),
          "model.language_model.layers.0.mlp.experts.down_proj": torch.randn(E, F, H),
          "model.language_model.layers.0.mlp.gate.weight": torch.randn(E, H)}
    src = tmp_path / "hf"
    hfio.save_sharded(hf, str(src))
    json.dump({"text_config": {"num_experts": E}}, open(src / "config.json", "w"))
    assert mm_convert(["Qwen3VLConverter", "hf_to_dcp", "--cfg.hf_dir", str(src), "--cfg.dcp_dir", str(tmp_path / "dcp")]) == 0
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.format_utils import dcp_to_torch_save
    dcp_to_torch_save(str(tmp_path / "dcp" / "release"), str(tmp_path / "flat.pt"))
    flat = torch.load(tmp_path / "flat.pt", weights_only=False)["model"]
    assert flat["model.model.language_model.layers.0.mlp.experts.gate_up_proj"].shape == (E * H, 2 * F)
    assert mm_convert(["Qwen3VLConverter", "dcp_to_hf", "--cfg.load_dir", str(tmp_path / "dcp"), "--cfg.save_dir",
                       str(tmp_path / "back"), "--cfg.model_assets_dir", str(src)]) == 0
    back = hfio.load_state_dict(str(tmp_path / "back"))
    assert set(back) == set(hf) and all(torch.equal(back[k], hf[k]) for k in hf)
    assert (tmp_path / "back" / "config.json").exists()
    # per-expert <-> fused
    assert mm_convert(["Qwen3VLConverter", "moe_expert", "--cfg.style", "split", "--cfg.hf_dir", str(src), "--cfg.save_dir",
                       str(tmp_path / "split")]) == 0
    sp = hfio.load_state_dict(str(tmp_path / "split"))
    g = sp["model.language_model.layers.0.mlp.experts.2.gate_proj.weight"]
    assert g.shape == (F, H) and torch.equal(g, hf["model.language_model.layers.0.mlp.experts.gate_up_proj"][2, :, :F].t())
    assert mm_convert(["Qwen3VLConverter", "moe_expert", "--cfg.style", "merge", "--cfg.hf_dir", str(tmp_path / "split"),
                       "--cfg.save_dir", str(tmp_path / "merged")]) == 0
    mg = hfio.load_state_dict(str(tmp_path / "merged"))
    assert all(torch.equal(mg[k], hf[k]) for k in hf)


def test_mm_convert_prefix_renames_generic_dcp_and_lora_merge(tmp_path):
    """InternVL / Mistral3 converters rename the sub-model prefixes of older exports on the way into DCP; the generic
    converter keeps names; LoraConverter folds a PEFT adapter into its base checkpoint."""
    import json
    from safetensors.torch import save_file
    from torch.distributed.checkpoint.format_utils import dcp_to_torch_save
    torch.manual_seed(0)
    old = {"language_model.model.layers.0.self_attn.q_proj.weight": torch.randn(8, 8),
           "language_model.lm_head.weight": torch.randn(16, 8), "vision_tower.embeddings.cls_token": torch.randn(1, 1, 8),
           "multi_modal_projector.linear_1.weight": torch.randn(8, 32)}
    src = tmp_path / "old"
    hfio.save_sharded(old, str(src))
    for conv in ("InternVLConverter", "Mistral3Converter"):
        out = tmp_path / conv
        assert mm_convert([conv, "hf_to_dcp", "--cfg.hf_dir", str(src), "--cfg.dcp_dir", str(out)]) == 0
        dcp_to_torch_save(str(out / "release"), str(out / "flat.pt"))
        flat = torch.load(out / "flat.pt", weights_only=False)["model"]
        assert set(flat) == {"model.model.language_model.layers.0.self_attn.q_proj.weight", "model.lm_head.weight",
                             "model.model.vision_tower.embeddings.cls_token", "model.model.multi_modal_projector.linear_1.weight"}
    assert mm_convert(["GenericDcpConverter", "hf_to_dcp", "--cfg.hf_dir", str(src), "--cfg.dcp_dir", str(tmp_path / "g")]) == 0
    assert mm_convert(["GenericDcpConverter", "dcp_to_hf", "--cfg.load_dir", str(tmp_path / "g"), "--cfg.save_dir",
                       str(tmp_path / "gb")]) == 0
    back = hfio.load_state_dict(str(tmp_path / "gb"))
    assert set(back) == set(old) and all(torch.equal(back[k], old[k]) for k in old)
    # LoRA merge
    base = {"model.layers.0.self_attn.q_proj.weight": torch.randn(8, 8), "model.norm.weight": torch.ones(8)}
    bdir, ldir = tmp_path / "base", tmp_path / "lora"
    hfio.save_sharded(base, str(bdir))
    json.dump({"model_type": "qwen3"}, open(bdir / "config.json", "w"))
    ldir.mkdir()
    A, B = torch.randn(2, 8), torch.randn(8, 2)
    save_file({"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": A,
               "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": B}, str(ldir / "adapter_model.safetensors"))
    json.dump({"r": 2, "lora_alpha": 4.0, "target_modules": ["q_proj"]}, open(ldir / "adapter_config.json", "w"))
    assert mm_convert(["LoraConverter", "merge_lora_to_base", "--cfg.base_dir", str(bdir), "--cfg.lora_dir", str(ldir),
                       "--cfg.save_dir", str(tmp_path / "merged_lora")]) == 0
    mg = hfio.load_state_dict(str(tmp_path / "merged_lora"))
    want = base["model.layers.0.self_attn.q_proj.weight"] + 2.0 * (B @ A)
    assert torch.allclose(mg["model.layers.0.self_attn.q_proj.weight"], want, atol=1e-6)
    assert torch.equal(mg["model.norm.weight"], base["model.norm.weight"]) and (tmp_path / "merged_lora" / "config.json").exists()
