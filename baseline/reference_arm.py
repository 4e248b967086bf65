"""The reference arm of the benchmark: the unmodified reference package (``baseline/_ref``) driven through its
own native trainer, ``ConfigManager(Arguments).load_and_parse()`` -> ``Trainer(args)`` -> ``train()``
(mindspeed_mm/fsdp/train/trainer.py:473-477), on the workload of the repository's own arm.

Nothing of this repository's models, kernels or engine is imported here.  What is supplied from outside the
reference: stand-ins for third-party symbols that are not installed (``baseline/shims``), a Hugging Face
``config.json`` of the model (the reference builds the stock ``transformers`` class named in it on the meta
device: mindspeed_mm/fsdp/models/modelhub.py:60-83), a YAML recipe in the reference's native schema, and a synthetic
dataset registered through the reference's ``data_register`` (``baseline/mm_ref_plugins``).

Timing: the dataset's fetch hook records CUDA events at iteration boundaries of the reference's own loop (every
iteration of that loop starts with barrier + synchronize, mindspeed_mm/fsdp/train/train_engine.py:259), so K whole
iterations -- forward, backward, gradient clipping call, optimizer step, loss read-back -- lie between two events.
Two regions: batches resident on the device, then batches copied from pinned host memory every step.
"""
from __future__ import annotations

import json
import os
import socket
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def qwen2_5_vl_hf_config(tiny: bool) -> dict:
    """config.json of Qwen2.5-VL-7B-Instruct (or a 2-layer miniature with the same structure)."""
    text = dict(
        model_type="qwen2_5_vl_text", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
        num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, hidden_act="silu",
        max_position_embeddings=128000, rms_norm_eps=1e-6, rope_theta=1000000.0, attention_dropout=0.0,
        use_sliding_window=False, sliding_window=32768, max_window_layers=28, tie_word_embeddings=False,
        rope_scaling={"type": "mrope", "mrope_section": [16, 24, 24]}, use_cache=False, initializer_range=0.02)
    vision = dict(
        model_type="qwen2_5_vl", depth=32, hidden_size=1280, hidden_act="silu", intermediate_size=3420, num_heads=16,
        in_chans=3, out_hidden_size=3584, patch_size=14, spatial_merge_size=2, spatial_patch_size=14,
        window_size=112, fullatt_block_indexes=[7, 15, 23, 31], tokens_per_second=2, temporal_patch_size=2)
    if tiny:
        text.update(vocab_size=32000, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, max_window_layers=2,
                    rope_scaling={"type": "mrope", "mrope_section": [8, 12, 12]})
        vision.update(depth=2, hidden_size=128, intermediate_size=256, num_heads=4, out_hidden_size=256,
                      fullatt_block_indexes=[1])
    cfg = dict(
        architectures=["Qwen2_5_VLForConditionalGeneration"], model_type="qwen2_5_vl",
        image_token_id=151655 if not tiny else 31999, video_token_id=151656 if not tiny else 31998,
        vision_start_token_id=151652 if not tiny else 31997, vision_end_token_id=151653 if not tiny else 31996,
        text_config=text, vision_config=vision, tie_word_embeddings=False, torch_dtype="bfloat16")
    # flat copies of the text keys: older releases of the config class read them at the top level
    for k, v in text.items():
        if k != "model_type":
            cfg.setdefault(k, v)
    return cfg


def recipe_yaml(model_dir: str, train_iters: int, attn: str) -> dict:
    """Native-schema recipe: FSDP2 over all ranks, bf16 parameters / fp32 reduction, full recompute of the ViT
    blocks and decoder layers, AdamW lr 1e-5 without clipping, micro-batch 1 (= one packed 8192-token batch)."""
    return dict(
        parallel=dict(
            tensor_parallel_size=1, fully_shard_parallel_size="auto",
            fsdp_plan=dict(apply_modules=["model.visual.blocks.{*}", "model.visual.merger", "model.visual",
                                          "model.language_model.embed_tokens", "model.language_model.layers.{*}",
                                          "model.language_model", "lm_head"],
                           param_dtype="bf16", reduce_dtype="fp32"),
            ring_attention_size=1, ulysses_parallel_size=1, expert_parallel_size=1),
        data=dict(
            dataset_param=dict(dataset_type="synthetic_packed_vlm",
                               preprocess_parameters=dict(model_name_or_path=model_dir),
                               basic_parameters=dict(dataset=model_dir, cutoff_len=8192)),
            dataloader_param=dict(pin_memory=False, shuffle=False, dataloader_mode="sampler", drop_last=True,
                                  sampler_type="BaseRandomBatchSampler", num_workers=0,
                                  collate_param=dict(model_name="qwen2_5vl"), enable_preload=False)),
        model=dict(model_name_or_path=model_dir, trust_remote_code=False, attn_implementation=attn, freeze=[]),
        features=dict(
            loss_cfg=dict(loss_type="default", router_aux_loss_coef=0.0),
            recompute=True,
            recompute_plan=dict(apply_modules=["model.visual.blocks.{*}", "model.language_model.layers.{*}"]),
            enable_chunk_loss=False),
        training=dict(
            micro_batch_size=1, gradient_accumulation_steps=1, seed=42, lr=1.0e-5, lr_decay_style="constant",
            lr_warmup_ratio=0.0, weight_decay=0.0, train_iters=train_iters, clip_grad=0.0,
            init_model_with_meta_device=True, optimizer="adamw", adam_fused=True, save_interval=10 ** 9,
            log_interval=10 ** 9, use_deter_comp=False, plugin=["mm_ref_plugins"]),
        tools=dict(profile=dict(enable=False), memory_profile=dict(enable=False)))


WAN_UNAVAILABLE = (
    "reference cannot train Wan through a stock path on this image: its Megatron entry point (pretrain_sora.py) needs "
    "the megatron and mindspeed packages, and its native Wan2.2 container imports names this snapshot does not define "
    "(ImportError: cannot import name 'GenerativeBaseModel' from mindspeed_mm.fsdp.models.base_model; "
    "mindspeed_mm.fsdp.train.generative_pipeline is absent)")


def run(args, clock_sampler_cls=None) -> int:
    import torch
    import yaml

    tiny = args.model == "tiny"
    if getattr(args, "workload", "vlm") != "vlm":
        if int(os.environ.get("RANK", "0")) == 0:
            why = WAN_UNAVAILABLE if args.workload == "wan" else "the reference arm covers the default (VLM) workload only"
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(_free_port()))
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])

    def unavailable(why: str) -> int:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    ref_dir = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "mindspeed_mm")):
        return unavailable("reference not installed under baseline/_ref (pip install --no-index --no-deps --target "
                           "baseline/_ref /root/reference)")
    for p in (HERE, ref_dir, os.path.join(HERE, "shims")):
        sys.path.insert(0, p)
    cuda = torch.cuda.is_available()
    seq = args.seq_len if not tiny else 1024
    if tiny:
        os.environ.update(MM_REF_SEQ_LEN=str(seq), MM_REF_SAMPLES="1", MM_REF_IMAGES="2", MM_REF_IMAGE_SIZE="224",
                          MM_REF_VOCAB="32000", MM_REF_IMAGE_TOKEN="31999", MM_REF_VISION_START="31997")
    else:
        os.environ.update(MM_REF_SEQ_LEN=str(seq), MM_REF_SAMPLES="4", MM_REF_IMAGES="2", MM_REF_IMAGE_SIZE="448")

    # The top-level package of the reference imports its Megatron patches unless this variable says "true"; the
    # native sub-package, read next, applies its torch-FSDP monkey patch when it says "true", and that patch
    # refuses every torch release except 2.7.1 and 2.9.0 (mindspeed_mm/fsdp/ops/fully_shard/fully_shard.py:840-847).
    # So: "true" for the first import, then off; the reference then shards with the stock
    # torch.distributed.fsdp.fully_shard.  Its attention registration (the other half of that patch function) does
    # work on this torch, and is applied through the reference's own function below.
    os.environ["NON_MEGATRON"] = "true"
    try:
        import mindspeed_mm  # noqa: F401
        os.environ["NON_MEGATRON"] = "false"
        from mindspeed_mm.config.config_manager import ConfigManager
        from mindspeed_mm.fsdp.ops.flash_attn.flash_attn import apply_transformers_attention_patch
        from mindspeed_mm.fsdp.params.argument import Arguments
        from mindspeed_mm.fsdp.train.trainer import Trainer
    except Exception as e:  # noqa: BLE001
        return unavailable(f"reference trainer import failed: {type(e).__name__}: {str(e).splitlines()[0][:200]}")
    if cuda:
        apply_transformers_attention_patch()
    else:                       # CPU dry run of the plumbing (development only): gloo, eager attention
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.accelerator.set_device_index = lambda index: None     # no accelerator to select on a CPU box

    warmup, steps = max(args.warmup, 3), args.steps
    work = tempfile.mkdtemp(prefix=f"mm_ref_r{rank}_")
    model_dir = os.path.join(work, "qwen2_5_vl")
    os.makedirs(model_dir)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(qwen2_5_vl_hf_config(tiny), f)
    from mm_ref_plugins.synthetic_vlm import PROBE
    PROBE.plan(warmup, steps)
    cfg_path = os.path.join(work, "recipe.yaml")
    with open(cfg_path, "w") as f:
        yaml.safe_dump(recipe_yaml(model_dir, PROBE.total_fetches, "flash_attention_2" if cuda else "sdpa"), f)

    sampler = clock_sampler_cls(local) if (clock_sampler_cls is not None and cuda) else None
    if sampler is not None:
        PROBE.on_mark["dev0"] = sampler.start
    sys.argv = [sys.argv[0], cfg_path]
    real_stdout, sys.stdout = sys.stdout, sys.stderr     # the reference prints its config and log to stdout
    try:
        ref_args = ConfigManager(Arguments).load_and_parse()
        trainer = Trainer(ref_args)
        n_params = sum(p.numel() for p in trainer.model.parameters())
        trainer.train()
    except Exception as e:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        msg = f"{type(e).__name__}: {str(e).splitlines()[0][:300] if str(e) else ''}"
        if sampler is not None and sampler.is_alive():
            sampler.stop()
        return unavailable(f"reference stock path failed at N={world}: {msg}")
    finally:
        sys.stdout = real_stdout
    clocks = sampler.stop() if sampler is not None else None

    import torch.distributed as dist
    ms = torch.tensor([PROBE.elapsed_ms("dev0", "dev1") / steps, PROBE.elapsed_ms("e2e0", "e2e1") / steps],
                      device="cuda" if cuda else "cpu")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = float(ms[0]), float(ms[1])
    ds = trainer.train_dataloader.dataset
    if rank == 0:
        tokens = seq * world
        out = {
            "metric": "Qwen2.5-VL-7B FSDP2 tokens/s", "value": round(tokens / (ms_dev / 1e3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_dev, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random-init weights, random text ids, U[0,1] images CLIP-normalised)",
            "impl": "reference",
            "config": {"model": "Qwen2.5-VL-7B" if not tiny else "tiny", "global_batch": world, "seq_len": seq,
                       "parallelism": f"fsdp{world}" if world > 1 else "single", "tokens_per_gpu": seq,
                       "images_per_gpu": 8 if not tiny else 2, "parameters": n_params,
                       "recompute": "activation checkpointing: every ViT block and decoder layer recomputed",
                       "optimizer": "torch AdamW fused, fp32 sharded parameters", "trainable": "all parameters",
                       "l2": "inputs_larger_than_L2 (weights + optimizer state are streamed every step)",
                       "path": "reference Trainer(args).train(): stock torch fully_shard, transformers "
                               "Qwen2_5_VLForConditionalGeneration, flash-attn 2 through the reference's attention "
                               "registration; its torch-FSDP monkey patch is not applied (refuses torch "
                               + torch.__version__ + ")",
                       "note": "value: batches resident on the device; every iteration of the reference loop "
                               "ends with barrier + synchronize and reads the loss back (loss.item())"},
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1) if cuda else None,
            "clocks": clocks,
            "e2e": {"value": round(tokens / (ms_e2e / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 2),
                    "h2d_bytes_per_step": ds.nbytes(), "d2h_bytes_per_step": 4},
            "gpu_launches": 0,
            "wan": {"unavailable": WAN_UNAVAILABLE},
        }
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0
