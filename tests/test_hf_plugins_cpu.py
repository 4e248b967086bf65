"""transformers classes on this package's ops and engine: the kernel plugin leaves logits unchanged and restores the
classes when removed; the adapter trains a stock ``Qwen3ForCausalLM`` / ``Qwen2_5_VLForConditionalGeneration`` under
the ZeRO-3 engine with the same parameters after two steps as plain autograd + AdamW."""
import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")

from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig  # noqa: E402
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.plugins import hf_kernels  # noqa: E402
from mindspeed_mm_b200.plugins.hf_adapter import HFModelAdapter  # noqa: E402


def _qwen3(attn="sdpa", moe=False):
    if moe:
        from transformers import Qwen3MoeConfig as C, Qwen3MoeForCausalLM as M
        extra = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=1, mlp_only_layers=[])
    else:
        from transformers import Qwen3Config as C, Qwen3ForCausalLM as M
        extra = {}
    cfg = C(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            head_dim=16, vocab_size=200, tie_word_embeddings=False, **extra)
    cfg._attn_implementation = attn
    torch.manual_seed(0)
    return M(cfg).float()


def test_kernel_plugin_keeps_logits_and_is_removable():
    from transformers.models.qwen3 import modeling_qwen3 as mq
    orig = (mq.Qwen3RMSNorm.forward, mq.Qwen3MLP.forward, mq.apply_rotary_pos_emb)
    base = _qwen3().eval()
    ids = torch.randint(0, 200, (2, 12))
    with torch.no_grad():
        want = base(input_ids=ids).logits
    rec = hf_kernels.apply_kernel_plugin(("qwen3", "qwen3_moe", "qwen2_5_vl", "not_a_family"))
    try:
        assert {"Qwen3RMSNorm", "Qwen3MLP", "apply_rotary_pos_emb"} <= set(rec["modeling_qwen3"])
        assert rec["attention"] == ["mm_b200", "mm_b200_flash"] and "modeling_not_a_family" not in rec
        assert mq.Qwen3RMSNorm.forward is not orig[0]
        patched = _qwen3("mm_b200").eval()
        patched.load_state_dict(base.state_dict())
        with torch.no_grad():
            got = patched(input_ids=ids).logits
            assert (got - want).abs().max() < 2e-5
            # right-padded batch: the padding mask reaches the attention function
            mask = torch.ones_like(ids)
            mask[1, 8:] = 0
            a = base(input_ids=ids, attention_mask=mask).logits
            b = patched(input_ids=ids, attention_mask=mask).logits
            assert (a[0] - b[0]).abs().max() < 2e-5 and (a[1, :8] - b[1, :8]).abs().max() < 2e-5
            # generation with the key / value cache
            g0 = base.generate(ids[:1], max_new_tokens=5, do_sample=False)
            g1 = patched.generate(ids[:1], max_new_tokens=5, do_sample=False)
            assert torch.equal(g0, g1)
    finally:
        hf_kernels.remove_kernel_plugin()
    assert (mq.Qwen3RMSNorm.forward, mq.Qwen3MLP.forward, mq.apply_rotary_pos_emb) == orig


def _two_steps(ref, batch_fn, loss_fn):
    """Plain autograd + AdamW on ``ref`` and the engine on a copy; returns (reference params, engine params).  A large
    Adam epsilon keeps entries whose gradient is rounding noise from moving by a full step in a random direction."""
    net = copy.deepcopy(ref)
    adapter = HFModelAdapter(net)
    eng = FSDPEngine(adapter.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=1e-3, eps=1e-4))
    adapter.attach(eng)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.0, eps=1e-4)
    for step in range(2):
        batch = batch_fn(step)
        opt.zero_grad()
        loss_fn(ref, batch).backward()
        opt.step()
        eng.set_lr(1e-3)
        ls, n = adapter(batch)
        (ls / n).backward()
        eng.end_micro_step()
        eng.finish_step()
    got = {k[len("model."):]: v for k, v in eng.named_full_params()}
    return dict(ref.named_parameters()), got


@pytest.mark.parametrize("moe", [False, True])
def test_adapter_trains_stock_causal_lm(moe):
    ref = _qwen3(moe=moe)

    def batch_fn(step):
        g = torch.Generator().manual_seed(step)
        ids = torch.randint(0, 200, (30,), generator=g)
        labels = torch.roll(ids, -1)
        labels[[13, 29]] = -100
        return dict(input_ids=ids, labels=labels, cu_seqlens=torch.tensor([0, 14, 30], dtype=torch.int32), max_seqlen=16)

    def loss_fn(model, b):
        # the same two sequences as separate rows
        ids, lab = b["input_ids"], b["labels"]
        rows = [(ids[:14], lab[:14]), (ids[14:], lab[14:])]
        tot, n = 0.0, 0
        for i, l in rows:
            logits = model(input_ids=i[None]).logits[0].float()
            tot = tot + torch.nn.functional.cross_entropy(logits, l, ignore_index=-100, reduction="sum")
            n += int((l != -100).sum())
        return tot / n

    want, got = _two_steps(ref, batch_fn, loss_fn)
    assert set(want) == set(got)
    for k in want:
        assert torch.allclose(got[k], want[k], atol=3e-5), (k, float((got[k] - want[k]).abs().max()))


def test_adapter_units_cover_every_parameter_once():
    model = _qwen3()
    adapter = HFModelAdapter(model)
    units = adapter.fsdp_units()
    names = [n for n, _ in units]
    assert "model.model.layers.0" in names and "model.model.embed_tokens" in names and "model.lm_head" in names
    seen = [id(p) for _, m in units for p in m.parameters()]
    assert len(seen) == len(set(seen)) == len(list(model.parameters()))
    # a tied head is untied so that the two modules can live in different units
    from transformers import Qwen3Config, Qwen3ForCausalLM
    tied = Qwen3ForCausalLM(Qwen3Config(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                                        num_key_value_heads=1, head_dim=16, vocab_size=50, tie_word_embeddings=True))
    assert tied.lm_head.weight is tied.model.embed_tokens.weight
    HFModelAdapter(tied)
    assert tied.lm_head.weight is not tied.model.embed_tokens.weight and torch.equal(tied.lm_head.weight, tied.model.embed_tokens.weight)


def test_adapter_trains_stock_vlm():
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=14,
               spatial_merge_size=2, temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1], in_channels=3)
    txt = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=300, rope_parameters=dict(rope_type="default", rope_theta=1e4, mrope_section=[2, 3, 3]),
               tie_word_embeddings=False)
    cfg = Qwen2_5_VLConfig(vision_config=vis, text_config=txt, image_token_id=290, video_token_id=291,
                           vision_start_token_id=292, vision_end_token_id=293)
    torch.manual_seed(0)
    ref = Qwen2_5_VLForConditionalGeneration(cfg).float()
    grid = torch.tensor([[1, 4, 4]])
    n_img = 4

    def batch_fn(step):
        g = torch.Generator().manual_seed(step)
        ids = torch.cat([torch.randint(0, 280, (4,), generator=g), torch.tensor([292]), torch.full((n_img,), 290),
                         torch.tensor([293]), torch.randint(0, 280, (6,), generator=g)])
        labels = torch.roll(ids, -1)
        labels[:10] = -100
        labels[-1] = -100
        return dict(input_ids=ids, labels=labels, pixel_values=torch.randn(16, 3 * 2 * 14 * 14, generator=g),
                    image_grid_thw=grid, mm_token_type_ids=(ids == 290).int()[None],
                    cu_seqlens=torch.tensor([0, ids.numel()], dtype=torch.int32), max_seqlen=ids.numel())

    def loss_fn(model, b):
        logits = model(input_ids=b["input_ids"][None], pixel_values=b["pixel_values"], image_grid_thw=grid,
                       mm_token_type_ids=b["mm_token_type_ids"]).logits[0].float()
        lab = b["labels"]
        return torch.nn.functional.cross_entropy(logits, lab, ignore_index=-100, reduction="sum") / (lab != -100).sum()

    net = copy.deepcopy(ref)
    adapter = HFModelAdapter(net)
    names = [n for n, _ in adapter.fsdp_units()]
    assert "model.model.visual.blocks.0" in names and "model.model.language_model.layers.1" in names
    want, got = _two_steps(ref, batch_fn, loss_fn)
    assert set(want) == set(got)
    for k in want:
        assert torch.allclose(got[k], want[k], atol=3e-5), (k, float((got[k] - want[k]).abs().max()))


def test_trainer_runs_a_stock_transformers_checkpoint(tmp_path, capsys):
    """``model_id: hf_auto``: config.json names the architecture, the safetensors load by name, three steps lower the loss
    of a fixed batch, and the ``save_format: hf`` output loads back into the stock class."""
    import os
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=14,
               spatial_merge_size=2, temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1], in_channels=3)
    txt = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=400, rope_parameters=dict(rope_type="default", rope_theta=1e4, mrope_section=[2, 3, 3]),
               tie_word_embeddings=False)
    cfg = Qwen2_5_VLConfig(vision_config=vis, text_config=txt, image_token_id=393, video_token_id=394,
                           vision_start_token_id=390, vision_end_token_id=391)
    torch.manual_seed(0)
    hf = Qwen2_5_VLForConditionalGeneration(cfg).float()
    src = tmp_path / "hf_in"
    hf.save_pretrained(src, safe_serialization=True)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = load_config(os.path.join(root, "examples/qwen2.5vl/tiny_hf_auto.yaml"),
                       [f"model.model_name_or_path={src}", "training.train_iters=3", f"training.save={tmp_path}/out",
                        "training.save_format=hf", "data.dataset_param.basic_parameters.num_samples=1"], world_size=1)
    try:
        tr = Trainer(args, device="cpu")
        assert type(tr.model.model).__name__ == "Qwen2_5_VLForConditionalGeneration"
        got = {k[len("model."):]: v for k, v in tr.engine.named_full_params()}
        for k, v in hf.state_dict().items():
            assert torch.allclose(got[k].float(), v, atol=1e-6), k
        hist = tr.train()
    finally:
        hf_kernels.remove_kernel_plugin()
    losses = [h["loss"] for h in hist] if hist and isinstance(hist[0], dict) else list(hist)
    assert losses[-1] < losses[0]
    back = Qwen2_5_VLForConditionalGeneration.from_pretrained(tmp_path / "out" / "hf", dtype=torch.float32)
    moved = sum(float((v - hf.state_dict()[k]).abs().max()) > 0 for k, v in back.state_dict().items())
    assert set(back.state_dict()) == set(hf.state_dict()) and moved > 10


def test_verl_plugin_entry_point(monkeypatch):
    from mindspeed_mm_b200.plugins import verl as vp
    monkeypatch.setenv("DETERMINISTIC", "1")
    try:
        rec = vp.apply_verl_plugin()
        assert "Qwen2_5_VLRMSNorm" in rec["modeling_qwen2_5_vl"] and "Qwen3VLMoeTextMLP" in rec["modeling_qwen3_vl_moe"]
        assert rec["attention"] == ["mm_b200", "mm_b200_flash"] and torch.are_deterministic_algorithms_enabled()
        a = torch.rand(3) + torch.rand(3)          # the generator has moved on since the plugin seeded it
        vp.seed_all(1234)
        b = torch.rand(3)
        vp.seed_all(1234)
        assert torch.equal(b, torch.rand(3)) and not torch.equal(a, b)
    finally:
        hf_kernels.remove_kernel_plugin()
        torch.use_deterministic_algorithms(False)


def test_zoo_id_with_a_checkpoint_runs_the_stock_architecture(tmp_path):
    """``model_id: mistral3`` is a switch setting of the composable model until it is pointed at a checkpoint directory:
    then the architecture config.json names (stock Mistral3ForConditionalGeneration: Pixtral tower + Mistral decoder) is
    built, its weights load by name, and text-only packs train it."""
    import os
    from transformers import Mistral3Config, Mistral3ForConditionalGeneration
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    cfg = Mistral3Config(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, image_size=56,
                           patch_size=14, head_dim=16),
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, vocab_size=1100, sliding_window=None), image_token_index=1023)
    torch.manual_seed(0)
    hf = Mistral3ForConditionalGeneration(cfg).float()
    src = tmp_path / "hf_in"
    hf.save_pretrained(src, safe_serialization=True)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = load_config(os.path.join(root, "examples/magistral-2509/tiny_native.yaml"),
                       [f"model.model_name_or_path={src}", "training.train_iters=3", "training.clip_grad=0.0",
                        "data.dataset_param.basic_parameters.images_per_sample=0",
                        "data.dataset_param.basic_parameters.num_samples=2", "data.dataloader_param.shuffle=false"], world_size=1)
    try:
        tr = Trainer(args, device="cpu")
        assert type(tr.model.model).__name__ == "Mistral3ForConditionalGeneration"
        got = {k[len("model."):]: v for k, v in tr.engine.named_full_params()}
        sd = hf.state_dict()
        assert set(got) == set(sd)
        for k, v in sd.items():
            assert torch.allclose(got[k].float(), v, atol=1e-6), k
        hist = tr.train()
    finally:
        hf_kernels.remove_kernel_plugin()
    losses = [float(h["loss"]) if isinstance(h, dict) else float(h) for h in hist]
    assert losses[-1] < losses[0]


def test_packed_rows_stay_separate_under_the_plugin_attention():
    """With the ``mm_b200`` attention implementation the adapter hands the sequence boundaries to the attention function:
    the logits of a packed row equal the logits of its sequences run one by one."""
    hf_kernels.apply_kernel_plugin(("qwen3",))
    try:
        model = _qwen3("mm_b200").eval()
        adapter = HFModelAdapter(model)
        ids = torch.randint(0, 200, (30,))
        with torch.no_grad():
            packed = adapter(dict(input_ids=ids, cu_seqlens=torch.tensor([0, 14, 30], dtype=torch.int32), max_seqlen=16))
            a = model(input_ids=ids[None, :14]).logits[0]
            b = model(input_ids=ids[None, 14:]).logits[0]
        assert (packed - torch.cat([a, b])).abs().max() < 2e-5
        with torch.no_grad():
            leaky = model(input_ids=ids[None]).logits[0]            # one long sequence: the second part sees the first
        assert (leaky[14:] - b).abs().max() > 1e-3
    finally:
        hf_kernels.remove_kernel_plugin()


def test_vision_tower_takes_the_packed_path_under_the_plugin():
    """``use_plugin_attention="packed_towers"`` puts the vision tower on the flash-named alias: its windows arrive as ONE varlen call per
    block (not one call per window) and the logits match the stock model's."""
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    vis = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, out_hidden_size=64, patch_size=14,
               spatial_merge_size=2, temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1], in_channels=3)
    txt = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=300, rope_parameters=dict(rope_type="default", rope_theta=1e4, mrope_section=[2, 3, 3]),
               tie_word_embeddings=False)
    cfg = Qwen2_5_VLConfig(vision_config=vis, text_config=txt, image_token_id=290, video_token_id=291,
                           vision_start_token_id=292, vision_end_token_id=293)
    torch.manual_seed(0)
    ref = Qwen2_5_VLForConditionalGeneration(cfg).float().eval()
    grid = torch.tensor([[1, 8, 8]])                        # 64 patches -> 4 windows of 16, 16 merged image tokens
    ids = torch.cat([torch.randint(0, 280, (4,)), torch.tensor([292]), torch.full((16,), 290), torch.tensor([293]),
                     torch.randint(0, 280, (6,))])
    batch = dict(input_ids=ids, pixel_values=torch.randn(64, 3 * 2 * 14 * 14), image_grid_thw=grid,
                 mm_token_type_ids=(ids == 290).int()[None])
    with torch.no_grad():
        want = ref(input_ids=ids[None], **{k: v for k, v in batch.items() if k != "input_ids"}).logits[0]
    hf_kernels.apply_kernel_plugin(("qwen2_5_vl",))
    calls = []
    orig = ops.attention_varlen
    try:
        net = copy.deepcopy(ref)
        adapter = HFModelAdapter(net, use_plugin_attention="packed_towers")
        assert net.config.vision_config._attn_implementation == hf_kernels.TOWER_ATTENTION_NAME
        ops.attention_varlen = lambda *a, **k: (calls.append(a[3].numel() - 1), orig(*a, **k))[1]
        with torch.no_grad():
            got = adapter(batch)
    finally:
        ops.attention_varlen = orig
        hf_kernels.remove_kernel_plugin()
    assert calls == [4, 1], calls                           # windowed block: 4 windows in one call; full block: 1 sequence
    assert (got - want).abs().max() < 3e-5
