"""Throughput of a STOCK transformers Qwen2.5-VL class trained through this package's plug-in path.

The modeling code is Hugging Face's own ``Qwen2_5_VLForConditionalGeneration``; ``plugins/hf_kernels.py`` substitutes the
sm_100a ops (RMSNorm, SwiGLU, rotary embedding, varlen attention) and ``plugins/hf_adapter.py`` puts its layers under the
flat-buffer ZeRO-3 engine.  The step is the one of the flagship benchmark: 8,192 packed tokens (4 samples, 2 images of
448 x 448 each), bf16 parameters, AdamW, full recompute.  One GPU:

    python benchmarks/bench_hf_auto.py --steps 4 --warmup 3 --no-plugin   # Qwen2.5-VL-7B, stock ops under the engine
    python benchmarks/bench_hf_auto.py --model tiny --steps 3           # CPU / smoke

Prints one JSON line with tokens/s and ms/step (CUDA events, inputs copied from pinned host memory every step).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def hf_config(tiny: bool) -> dict:
    """config.json of Qwen2.5-VL-7B-Instruct, or a 2-layer miniature of the same structure."""
    text = dict(model_type="qwen2_5_vl_text", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=128000,
                rms_norm_eps=1e-6, tie_word_embeddings=False,
                rope_parameters=dict(rope_type="default", rope_theta=1e6, mrope_section=[16, 24, 24]))
    vision = dict(model_type="qwen2_5_vl", depth=32, hidden_size=1280, hidden_act="silu", intermediate_size=3420,
                  num_heads=16, in_chans=3, out_hidden_size=3584, patch_size=14, spatial_merge_size=2,
                  temporal_patch_size=2, window_size=112, fullatt_block_indexes=[7, 15, 23, 31])
    ids = dict(image_token_id=151655, video_token_id=151656, vision_start_token_id=151652, vision_end_token_id=151653)
    if tiny:
        text.update(vocab_size=32000, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, rope_parameters=dict(rope_type="default", rope_theta=1e6, mrope_section=[8, 12, 12]))
        vision.update(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, out_hidden_size=256,
                      fullatt_block_indexes=[1])
        ids = dict(image_token_id=31999, video_token_id=31998, vision_start_token_id=31997, vision_end_token_id=31996)
    return dict(model_type="qwen2_5_vl", text_config=text, vision_config=vision, tie_word_embeddings=False, **ids)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2_5_vl_7b", choices=["qwen2_5_vl_7b", "tiny"])
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--no-plugin", action="store_true", help="stock modeling code with its own ops (sdpa attention)")
    args = ap.parse_args()

    from mindspeed_mm_b200 import ops
    from mindspeed_mm_b200.api import stable_init_fn
    from mindspeed_mm_b200.data.collate import PackedVLMCollator, batch_nbytes, to_device
    from mindspeed_mm_b200.data.synthetic import SyntheticVLMDataset, SyntheticVLMSpec
    from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig
    from mindspeed_mm_b200.plugins.hf_auto import HFAutoConfig, HFAutoModel

    tiny = args.model == "tiny"
    cuda = torch.cuda.is_available()
    if cuda and not tiny and not args.no_plugin:
        # The full-size model with the plug-in ended in "illegal memory access" inside the vision tower's first blocks on
        # a B200 (the miniature and the full-size model without the plug-in run clean).  Until the faulting launch has been
        # found by reading, this combination stays off the GPU.
        raise SystemExit("qwen2_5_vl_7b with the kernel plug-in is closed on the GPU (unresolved memory fault); "
                         "run --model tiny, or --no-plugin")
    dev = torch.device("cuda:0" if cuda else "cpu")
    with torch.device("meta"):
        model = HFAutoModel(HFAutoConfig(hf=hf_config(tiny), kernel_plugin=not args.no_plugin))
    engine = FSDPEngine(model.fsdp_units(), group=False, device=dev,
                        param_dtype=torch.bfloat16 if cuda else torch.float32,
                        opt=OptimConfig(lr=1e-5, weight_decay=0.0, clip_grad=0.0), recompute=True)
    model.attach(engine, materialize=False)
    engine.materialize(stable_init_fn(0.02, 0))

    cfg = model.config
    seq = args.seq_len if not tiny else 1024
    per = seq // (4 if not tiny else 1)
    ds = SyntheticVLMDataset(SyntheticVLMSpec(
        seq_len=per, images_per_sample=2, image_size=448 if not tiny else 224, vocab_size=cfg.text.vocab_size,
        image_token_id=cfg.image_token_id, vision_start_token_id=cfg.vision_start_token_id, seed=1234,
        pixel_dtype=torch.bfloat16 if cuda else torch.float32, patch=cfg.vision.patch_size,
        merge=cfg.vision.spatial_merge_size))
    col = PackedVLMCollator.for_config(cfg, pixel_dtype=torch.bfloat16 if cuda else torch.float32, pin=cuda)
    n_pack = 4 if not tiny else 1
    host = [col([ds[b * n_pack + i] for i in range(n_pack)]) for b in range(4)]

    def step(i):
        b = to_device(host[i % len(host)], dev)
        engine.set_lr(1e-5)
        loss_sum, n = model(b)
        loss = loss_sum / n
        loss.backward()
        engine.end_micro_step()
        engine.finish_step()
        return float(loss.detach())                                   # device -> host read of the step's loss

    for i in range(args.warmup):
        last = step(i)
    if cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for i in range(args.steps):
        last = step(args.warmup + i)
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    else:
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
    tokens = host[0]["n_tokens"]
    print(json.dumps({
        "metric": "stock transformers Qwen2.5-VL through the kernel plug-in and ZeRO-3 engine, tokens/s",
        "value": round(tokens / (ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 2), "steps": args.steps,
        "warmup": args.warmup, "model": args.model, "plugin": not args.no_plugin, "seq_len": seq, "loss": round(last, 4),
        "h2d_bytes_per_step": batch_nbytes(host[0]), "library_fallbacks": ops.library_fallbacks(),
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1) if cuda else None}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
