"""Model families end to end on one GPU through the sharding engine (bf16, native op tier): two optimizer steps,
finite losses, no kernel reported a timed-out wait."""
import pytest
import torch

from mindspeed_mm_b200 import ops
from mindspeed_mm_b200.api import stable_init_fn
from mindspeed_mm_b200.parallel.fsdp import EngineMux, FSDPEngine, OptimConfig
from mindspeed_mm_b200.parallel.state import init_parallel_state, reset_parallel_state

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _vlm_batch(cfg, seq=512, img=224):
    from mindspeed_mm_b200.data.collate import PackedVLMCollator, to_device
    from mindspeed_mm_b200.data.synthetic import SyntheticVLMDataset, SyntheticVLMSpec
    ds = SyntheticVLMDataset(SyntheticVLMSpec(seq_len=seq, images_per_sample=1, image_size=img, vocab_size=cfg.text.vocab_size,
                                              image_token_id=cfg.image_token_id, vision_start_token_id=cfg.vision_start_token_id,
                                              pixel_dtype=torch.bfloat16, patch=cfg.vision.patch_size,
                                              merge=cfg.vision.spatial_merge_size))
    coll = PackedVLMCollator.for_config(cfg, pixel_dtype=torch.bfloat16)
    return to_device(coll([ds[0], ds[1]]), torch.device(DEV))


def _steps(model, eng, batch, n=2):
    losses = []
    for _ in range(n):
        eng.set_lr(1e-3)
        out = model(batch, run=eng.run)
        loss = out[0] / out[1] if isinstance(out, tuple) else out
        loss.backward()
        eng.end_micro_step()
        eng.finish_step()
        losses.append(float(loss.detach()))
    from mindspeed_mm_b200.ops import native
    native.check_status()
    assert all(l == l and abs(l) < 1e4 for l in losses), losses
    return losses


@pytest.fixture(autouse=True)
def _state():
    ops.set_tier("native")
    reset_parallel_state()
    init_parallel_state(world_size=1, device_type="cuda")
    yield
    reset_parallel_state()


def test_qwen3_5_gdn_hybrid_with_native_state_pass():
    """GDN layers at K = V = 128, chunk 64: the tcgen05 state-pass kernel and the conv1d / l2norm kernels are on the path."""
    from mindspeed_mm_b200.models.qwen3_5 import Qwen35Config, Qwen35Model
    cfg = Qwen35Config.tiny()
    t = cfg.text
    t.linear_key_head_dim = t.linear_value_head_dim = 128
    t.gdn_chunk = 64
    with torch.device("meta"):
        model = Qwen35Model(cfg)
    eng = FSDPEngine(model.fsdp_units(), group=False, device=DEV, param_dtype=torch.bfloat16, opt=OptimConfig(lr=1e-3))
    eng.materialize(stable_init_fn(0.02, 0))
    from mindspeed_mm_b200.ops import native
    before = native.LAUNCHES
    _steps(model, eng, _vlm_batch(cfg))
    assert native.LAUNCHES > before


def test_qwen3_vl_moe_native_experts():
    from mindspeed_mm_b200.models.qwen3_vl import Qwen3VLConfig, Qwen3VLModel
    cfg = Qwen3VLConfig.tiny()
    with torch.device("meta"):
        model = Qwen3VLModel(cfg, ep_size=1)
    ex = [p for _, m in model.expert_units() for p in m.parameters()]
    opt = OptimConfig(lr=1e-3)
    dense = FSDPEngine(model.fsdp_units(), group=False, device=DEV, param_dtype=torch.bfloat16, opt=opt, exclude_params=ex)
    expert = FSDPEngine(model.expert_units(), group=False, device=DEV, param_dtype=torch.bfloat16, opt=opt, no_recompute=())
    mux = EngineMux(dense, expert)
    mux.materialize(stable_init_fn(0.02, 0))
    _steps(model, mux, _vlm_batch(cfg, seq=384))


def test_wan_dit_and_mmdit():
    from mindspeed_mm_b200.models.diffusion import FlowMatchScheduler
    from mindspeed_mm_b200.models.mmdit import MMDiT, MMDiTConfig
    from mindspeed_mm_b200.models.wan import SoRAModel, WanConfig, WanDiT
    cfg = WanConfig.tiny()
    with torch.device("meta"):
        net = WanDiT(cfg)
    model = SoRAModel(net, FlowMatchScheduler(shift=5.0, sigma_min=0.0, extra_one_step=True), seed=0)
    eng = FSDPEngine(model.fsdp_units(), group=False, device=DEV, param_dtype=torch.bfloat16, opt=OptimConfig(lr=1e-3),
                     no_recompute=())
    eng.materialize(stable_init_fn(0.05, 0))
    batch = dict(latents=torch.randn(1, cfg.in_dim, 3, 16, 16, device=DEV, dtype=torch.bfloat16),
                 prompt=torch.randn(1, cfg.text_len, cfg.text_dim, device=DEV, dtype=torch.bfloat16))
    _steps(model, eng, batch)
    mc = MMDiTConfig.tiny()
    dit = MMDiT(mc).to(DEV, torch.bfloat16)
    for p in dit.parameters():
        torch.nn.init.normal_(p, std=0.02)
    y = dit(torch.randn(1, mc.in_channels, 1, 8, 8, device=DEV, dtype=torch.bfloat16), torch.tensor([500.0], device=DEV),
            torch.randn(1, 6, mc.text_dim, device=DEV, dtype=torch.bfloat16),
            torch.randn(1, mc.pooled_dim, device=DEV, dtype=torch.bfloat16), torch.tensor([3.5], device=DEV))
    y.float().pow(2).mean().backward()
    assert torch.isfinite(y).all()


def test_composable_presets_on_gpu():
    from mindspeed_mm_b200.data.collate import PackedVLMCollator, to_device
    from mindspeed_mm_b200.data.synthetic import SyntheticVLMDataset, SyntheticVLMSpec
    from mindspeed_mm_b200.models.composable import PRESETS, ComposableLM

    def _composable_batch(cfg):
        ds = SyntheticVLMDataset(SyntheticVLMSpec(seq_len=96, images_per_sample=1, image_size=56, vocab_size=1024,
                                                  image_token_id=1023, vision_start_token_id=1021,
                                                  temporal_patch=1 if cfg.vision_kind == "vit" else 2))
        b = PackedVLMCollator(1023, 1021, vit_head_dim=32)([ds[0], ds[1]])
        if cfg.vision_kind is None:
            b.pop("pixel_values")
        if cfg.audio is not None:
            b["audio_features"] = [torch.randn(16, 40)]
            b["input_ids"][5:15] = cfg.audio_token_id
        return b
    for mid in ("kimik2_5", "gemma4", "qwen3omni"):
        cfg = PRESETS[mid]
        torch.manual_seed(0)
        m = ComposableLM(cfg)
        m.init_weights(0)
        m = m.to(DEV, torch.bfloat16)
        b = to_device(_composable_batch(cfg), torch.device(DEV))
        if "pixel_values" in b:
            b["pixel_values"] = b["pixel_values"].to(torch.bfloat16)
        loss, n = m(b)
        (loss / n).backward()
        assert torch.isfinite(loss), mid


def test_internvl_and_stock_transformers_class_on_gpu():
    """InternVL (native model) against its fp32 CPU copy, and a stock transformers Qwen3 with the kernel plugin and the
    ``mm_b200`` attention implementation against the same class on stock kernels: bf16 on the GPU, no library fallback on
    the patched class."""
    from mindspeed_mm_b200.models.internvl import InternVLConfig, InternVLModel
    cfg = InternVLConfig.tiny()
    cfg.vision.hidden_size, cfg.vision.num_heads, cfg.vision.intermediate_size = 128, 2, 256      # head dim 64
    cfg.text.hidden_size, cfg.text.num_attention_heads, cfg.text.num_key_value_heads, cfg.text.head_dim = 128, 2, 1, 64
    cfg.text.intermediate_size = 256
    torch.manual_seed(0)
    ref_model = InternVLModel(cfg).float()
    ref_model.init_weights(0)
    g = torch.Generator().manual_seed(1)
    ids = torch.cat([torch.randint(0, 140, (9,), generator=g), torch.full((2 * cfg.tokens_per_tile,), cfg.image_token_id),
                     torch.randint(0, 140, (15,), generator=g)])
    labels = torch.roll(ids, -1)
    labels[ids == cfg.image_token_id] = -100
    batch = dict(input_ids=ids, labels=labels, pixel_values=torch.randn(2, 3, 56, 56, generator=g),
                 cu_seqlens=torch.tensor([0, ids.numel()], dtype=torch.int32), max_seqlen=ids.numel())
    ls, n = ref_model(batch)
    gpu = InternVLModel(cfg)
    gpu.load_state_dict(ref_model.state_dict())
    gpu = gpu.to(DEV, torch.bfloat16)
    from mindspeed_mm_b200.data.collate import to_device
    b = to_device(batch, torch.device(DEV))
    b["pixel_values"] = b["pixel_values"].to(torch.bfloat16)
    lg, ng = gpu(b)
    (lg / ng).backward()
    assert abs(float(lg / ng) - float(ls / n)) < 3e-2 * float(ls / n)
    assert all(torch.isfinite(p.grad).all() for p in gpu.parameters() if p.grad is not None)
    # stock class + plugin
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from mindspeed_mm_b200.plugins import hf_kernels
    hc = Qwen3Config(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=64, vocab_size=512, tie_word_embeddings=False)
    hc._attn_implementation = "sdpa"
    torch.manual_seed(0)
    base = Qwen3ForCausalLM(hc).to(DEV, torch.bfloat16).eval()
    x = torch.randint(0, 512, (2, 128), device=DEV)
    with torch.no_grad():
        want = base(input_ids=x).logits.float()
    hf_kernels.apply_kernel_plugin(("qwen3",))
    try:
        hc2 = Qwen3Config(**{k: v for k, v in hc.to_dict().items() if k in ("hidden_size", "intermediate_size", "num_hidden_layers",
                                                                       "num_attention_heads", "num_key_value_heads", "head_dim",
                                                                       "vocab_size", "tie_word_embeddings")})
        hc2._attn_implementation = "mm_b200"
        patched = Qwen3ForCausalLM(hc2).to(DEV, torch.bfloat16).eval()
        patched.load_state_dict(base.state_dict())
        ops.library_fallbacks(reset=True)
        with torch.no_grad():
            got = patched(input_ids=x).logits.float()
        assert not ops.library_fallbacks(), ops.library_fallbacks()
    finally:
        hf_kernels.remove_kernel_plugin()
    assert (got - want).abs().max() <= 5e-2 * want.abs().max()


def test_stock_transformers_checkpoint_trains_under_the_engine_on_gpu(tmp_path):
    """``model_id: hf_auto`` on the GPU: stock Qwen2.5-VL class built on the meta device, bf16 flat shards, recompute through
    the re-routed sub-module calls, the kernel plugin and the ``mm_b200`` attention implementation inside the class."""
    import os
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.plugins import hf_kernels
    from mindspeed_mm_b200.runtime.trainer import Trainer
    vis = dict(depth=2, hidden_size=128, intermediate_size=256, num_heads=2, out_hidden_size=256, patch_size=14,
               spatial_merge_size=2, temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1], in_channels=3)
    txt = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=512, rope_parameters=dict(rope_type="default", rope_theta=1e4, mrope_section=[8, 12, 12]),
               tie_word_embeddings=False)
    cfg = Qwen2_5_VLConfig(vision_config=vis, text_config=txt, image_token_id=503, video_token_id=504,
                           vision_start_token_id=500, vision_end_token_id=501)
    torch.manual_seed(0)
    src = tmp_path / "hf_in"
    Qwen2_5_VLForConditionalGeneration(cfg).float().save_pretrained(src, safe_serialization=True)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    args = load_config(os.path.join(root, "examples/qwen2.5vl/tiny_hf_auto.yaml"),
                       [f"model.model_name_or_path={src}", "training.train_iters=4", "training.lr=3e-3",
                        "data.dataset_param.basic_parameters.num_samples=1"], world_size=1)
    reset_parallel_state()
    try:
        tr = Trainer(args, device=DEV)
        assert type(tr.model.model).__name__ == "Qwen2_5_VLForConditionalGeneration"
        hist = tr.train()
    finally:
        hf_kernels.remove_kernel_plugin()
        reset_parallel_state()
    losses = [float(h["loss"]) if isinstance(h, dict) else float(h) for h in hist]
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses


def test_recompute_with_skipped_last_gemm_matches_graph_keeping_run():
    """The re-forward of a checkpointed block does not rerun its last GEMM (the value only feeds a residual add);
    one optimizer step must equal the step of the same model with autograd graphs kept."""
    from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel
    cfg = Qwen25VLConfig.tiny()
    batch = _vlm_batch(cfg)
    results = []
    for recompute in (True, False):
        with torch.device("meta"):
            model = Qwen25VLModel(cfg)
        eng = FSDPEngine(model.fsdp_units(), group=False, device=DEV, param_dtype=torch.bfloat16, opt=OptimConfig(lr=1e-3),
                         recompute=recompute)
        eng.materialize(stable_init_fn(0.02, 0))
        losses = _steps(model, eng, batch, n=2)
        results.append((losses, {n: t.detach().float().clone() for n, t in eng.named_full_params()}))
    (la, pa), (lb, pb) = results
    assert abs(la[0] - lb[0]) < 1e-3 and abs(la[1] - lb[1]) < 2e-2
    worst = max((pa[n] - pb[n]).abs().mean().item() for n in pa)
    assert worst < 3e-4, worst
