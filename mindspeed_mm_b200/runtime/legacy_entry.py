"""Shared body of the Megatron-style entry scripts (``pretrain_vlm.py``, ``pretrain_sora.py`` ...).

The reference's scripts each define ``model_provider / get_batch / loss_func / forward_step /
train_valid_test_datasets_provider`` and hand them to ``pretrain()`` (pretrain_vlm.py:35-269,
mindspeed_mm/training.py:86-346).  Here ``pretrain(kind)`` parses the same command line
(flags + ``--mm-model/--mm-data/--mm-tool``), builds the model from ``args.mm.model``, maps the Megatron
parallel flags onto the shared runtime (``--use-torch-fsdp2`` or plain data parallel -> sharding engine;
``--tensor-model-parallel-size`` / ``--pipeline-model-parallel-size`` -> the TP / PP backends) and runs the same
``TrainEngine`` loop as the native trainer, printing the same log line.
"""
from __future__ import annotations

import os
import sys
from typing import Optional

import torch
import torch.distributed as dist

from ..api import init_distributed, stable_init_fn
from ..config.legacy import parse_legacy_args
from ..parallel.fsdp import FSDPEngine, OptimConfig
from ..parallel.state import init_parallel_state
from .logging import print_rank0
from .loss import build_loss
from .lr_scheduler import LRSchedule
from .tools import Profiler
from .train_engine import TrainConfig, TrainEngine


def model_provider(kind: str, args):
    """Build the (meta-device) model named by ``args.mm.model``."""
    mm = args.mm.model.to_dict()
    if kind == "vlm":
        from ..models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel
        cfg = Qwen25VLConfig.from_mm_json(mm)
        with torch.device("meta"):
            model = Qwen25VLModel(cfg)
        ve = mm["image_encoder"]
        if ve["vision_encoder"].get("freeze", False):
            for n, p in model.visual.named_parameters():
                if not n.startswith("merger"):
                    p.requires_grad_(False)
        if ve["vision_projector"].get("freeze", False):
            for p in model.visual.merger.parameters():
                p.requires_grad_(False)
        return model
    if kind == "sora":
        from ..models.diffusion import build_scheduler
        from ..models.wan import SoRAModel, WanConfig, WanDiT
        pred = dict(mm["predictor"])
        if pred.get("model_id") != "wandit":
            from ..models.registry import build_model
            with torch.device("meta"):
                net = build_model(pred["model_id"], pred)
        else:
            with torch.device("meta"):
                net = WanDiT(WanConfig.from_mm_json(pred))
        from ..models.towers import build_ae, build_text_encoder
        ae = None if mm.get("load_video_features", True) else build_ae(mm.get("ae"))
        te = None if mm.get("load_text_features", True) else build_text_encoder(mm.get("text_encoder"))
        lora = mm.get("lora") or {}
        if lora.get("enable"):                       # adapters on the predictor's projections, everything else frozen
            from types import SimpleNamespace
            from ..tasks.lora import apply_lora
            apply_lora(net, SimpleNamespace(rank=int(lora.get("rank", 16)), alpha=float(lora.get("alpha", 16)),
                                            dropout=float(lora.get("dropout", 0.0)),
                                            target_modules=list(lora.get("target_modules") or [])))
        return SoRAModel(net, build_scheduler(mm.get("diffusion", {})), ae=ae, text_encoder=te, seed=args.seed,
                         prior_loss_weight=float(mm.get("prior_loss_weight", 1.0)))
    raise ValueError(f"unknown entry kind {kind}")


class _Namespace:
    """Attribute view of a dict (the dataset classes read ``dataset_param.basic_parameters`` etc.)."""

    def __init__(self, d: dict):
        self.__dict__.update(d)


def _real_dataset(data: dict, model):
    """The dataset that ``--mm-data`` names, when its type is registered and its files exist; None otherwise.
    ``dataset_type``: huggingface / multimodal (sharegpt conversations with images or video), feature (pre-extracted
    latents + prompt embeddings), t2v / i2v (raw video or image + caption); mindspeed_mm/data/__init__.py:30-95."""
    from ..data import data_register
    from ..data import multimodal as _mm   # noqa: F401  (registers huggingface / multimodal / feature / t2v / i2v)
    dp = data.get("dataset_param") or {}
    kind = dp.get("dataset_type")
    if not kind or kind.startswith("synthetic"):
        return None
    try:
        cls = data_register.get(kind)
    except KeyError:
        return None
    basic = dp.get("basic_parameters") or {}
    if kind == "dreambooth":                     # a folder of subject images, no index file
        if not os.path.isdir(basic.get("instance_data_dir") or ""):
            return None
        return cls(_Namespace(dict(dataset_type=kind, basic_parameters=basic,
                                   preprocess_parameters=dp.get("preprocess_parameters") or {})), model=model)
    src = basic.get("dataset") or basic.get("data_path") or basic.get("index")
    files = [src] if isinstance(src, str) else list(src or [])
    root = basic.get("dataset_dir") or basic.get("data_folder") or ""
    paths = [f if os.path.isabs(f) or not root or os.path.exists(f) else os.path.join(root, f) for f in files]
    if not paths or not all(os.path.exists(p) for p in paths):
        return None
    return cls(_Namespace(dict(dataset_type=kind, basic_parameters=basic,
                               preprocess_parameters=dp.get("preprocess_parameters") or {}, attr=dp.get("attr") or {})),
               model=model)


def datasets_provider(kind: str, args, model, ps, consumed_samples: int = 0):
    """Training batches for the legacy entry points.

    ``--mm-data`` decides: a registered ``dataset_type`` whose files exist is read for real (conversation json / jsonl
    through the chat template and the image processor, feature folders, raw video + captions); otherwise synthetic
    samples of the model's shapes are generated (no files needed: benchmarks, smoke tests).  ``dataloader_mode:
    dynamic_batching`` packs samples greedily up to ``--seq-length`` tokens per micro-batch
    (mindspeed_mm/data/dataloader/dynamic_batching_dataloader.py:37-159); ``consumed_samples`` (from a resumed
    checkpoint) fast-forwards the sampler (pretrain_vlm.py:217)."""
    from ..data.collate import PackedVLMCollator
    from ..data.samplers import BaseRandomBatchSampler
    from ..data.synthetic import (SyntheticVideoLatentDataset, SyntheticVideoLatentSpec, SyntheticVLMDataset,
                                  SyntheticVLMSpec)
    data = args.mm.data.to_dict() if hasattr(args.mm, "data") else {}
    basic = data.get("dataset_param", {}).get("basic_parameters", {})
    dl = data.get("dataloader_param") or {}
    real = _real_dataset(data, model)
    if kind == "vlm":
        cfg = model.config
        seq = int(args.seq_length or 1024)
        ds = real if real is not None else SyntheticVLMDataset(SyntheticVLMSpec(
            seq_len=seq, images_per_sample=int(basic.get("images_per_sample", 1)), image_size=int(basic.get("image_size", 224)),
            vocab_size=cfg.text.vocab_size, image_token_id=cfg.image_token_id,
            vision_start_token_id=cfg.vision_start_token_id, seed=args.seed, num_samples=int(basic.get("num_samples", 1 << 20)),
            patch=cfg.vision.patch_size, merge=cfg.vision.spatial_merge_size))
        coll = PackedVLMCollator.for_config(cfg)
    else:
        c = model.predictor.config
        channels = getattr(c, "in_dim", None) or getattr(c, "in_channels")       # Wan names it in_dim, the other DiTs in_channels
        ds = real if real is not None else SyntheticVideoLatentDataset(SyntheticVideoLatentSpec(
            channels=channels, frames=int(basic.get("frames", 5)), height=int(basic.get("height", 16)),
            width=int(basic.get("width", 16)), text_len=int(getattr(c, "text_len", basic.get("text_len", 16))),
            text_dim=c.text_dim, seed=args.seed,
            pooled_dim=int(c.pooled_dim) if getattr(model.predictor, "cond_input", "") == "added_cond" else 0,
            num_samples=int(basic.get("num_samples", 1 << 20))))
        coll = lambda ss: {k: torch.stack([s[k] for s in ss]) for k in ss[0]}   # noqa: E731
    shuffle = bool(dl.get("shuffle", True))
    if real is not None:
        print_rank0(f"> dataset: {type(ds).__name__} with {len(ds)} samples ({data['dataset_param'].get('dataset_type')})")
    if kind == "vlm" and dl.get("dataloader_mode") == "dynamic_batching":
        # one sample at a time from the sampler, packed greedily to at most `seq` tokens per micro-batch
        from ..data.packing import DynamicBatcher
        sampler = BaseRandomBatchSampler(len(ds), 1, ps.get_dp_rank(), ps.get_dp_world_size(), seed=args.seed,
                                         shuffle=shuffle, drop_last=bool(dl.get("drop_last", True)))
        sampler.consumed = int(consumed_samples)

        def samples():
            for idx in sampler:
                yield ds[idx[0]]

        def gen():
            for group in DynamicBatcher(samples(), seq, int(dl.get("dynamic_batch_buffer_size", 200))):
                yield coll(group)
        return gen()
    sampler = BaseRandomBatchSampler(len(ds), args.micro_batch_size, ps.get_dp_rank(), ps.get_dp_world_size(), seed=args.seed,
                                     shuffle=shuffle, drop_last=bool(dl.get("drop_last", True)))
    sampler.consumed = int(consumed_samples)

    def gen():
        for idx in sampler:
            yield coll([ds[i] for i in idx])
    return gen()


def pretrain(kind: str, argv=None, device: Optional[str] = None):
    args = parse_legacy_args(argv)
    dev, rank, world = init_distributed(device)
    from ..config.legacy import validate_args
    args.derived = validate_args(args, world)        # raises with the flags at fault before anything is built
    torch.manual_seed(args.seed)
    tp, pp, cp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size, args.context_parallel_size
    if tp > 1 or pp > 1:
        from ..parallel.mcore import pretrain_mcore
        return pretrain_mcore(kind, args, dev, rank, world)
    uly = cp if args.context_parallel_algo in ("ulysses_cp_algo", "hybrid_cp_algo") else 1
    if args.context_parallel_algo == "hybrid_cp_algo":
        uly = int(getattr(args, "ulysses_degree_in_cp", None) or cp)
    f2 = None
    if getattr(args, "fsdp2_config_path", None):
        from ..config.legacy import load_fsdp2_config
        f2 = load_fsdp2_config(args.fsdp2_config_path)
    elif getattr(args, "layerzero", False) and getattr(args, "layerzero_config", None):
        from ..config.legacy import load_layerzero_config          # same engine, LayerZero's key names
        f2 = load_layerzero_config(args.layerzero_config)
    shard = f2["sharding_size"] if f2 and f2["sharding_size"] not in (None, world) else None
    if shard and (shard > world or world % shard or shard % cp):
        print_rank0(f"fsdp2 config asks for sharding_size={shard}, which does not divide the {world} ranks of this job: "
                    f"sharding over all data ranks instead")
        shard = None
    ps = init_parallel_state(world_size=world, device_type=dev.type, ulysses_parallel_size=uly,
                             ring_attention_size=cp // uly,
                             fully_shard_parallel_size=(int(shard) // cp if shard else "auto"))
    model = model_provider(kind, args)
    # model.json "patch" block of the reference (mindspeed_mm/patchs/patch_manager.py): the entries that change training
    patch = (args.mm.model.to_dict().get("patch") or {}) if hasattr(args.mm, "model") else {}
    acg = patch.get("adaptive_clip_grad_norm") or {}
    ema_decay = float(acg.get("clip_grad_ema_decay", 0.99)) if (acg is True or acg) else 0.0
    opt = OptimConfig(lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                      weight_decay=args.weight_decay, clip_grad=args.clip_grad, clip_grad_ema_decay=ema_decay,
                      kind="muon" if (getattr(args, "optimizer", None) == "muon" or patch.get("muon_optimizer")) else "adamw")
    accum = max(1, args.global_batch_size // (args.micro_batch_size * ps.get_dp_world_size()))
    param_dtype = torch.bfloat16 if (args.bf16 and dev.type == "cuda") else torch.float32
    extra = {}
    if f2 is not None:
        if f2["param_dtype"] is not None and dev.type == "cuda":
            param_dtype = f2["param_dtype"]
        if f2["reduce_dtype"] is not None:
            extra["reduce_dtype"] = f2["reduce_dtype"]
        if world > 1 and ps.size("dp_replicate") > 1:         # sharding_size < ranks: hybrid sharding
            extra["replicate_group"] = ps.group("dp_replicate")
        if f2.get("offload_to_cpu"):
            extra["offload_optimizer"] = True
        if "prefetch" in f2:
            extra["prefetch"] = f2["prefetch"]
        if f2["unknown_keys"]:
            print_rank0(f"fsdp2 config keys without effect here: {f2['unknown_keys']}")
    engine = FSDPEngine(model.fsdp_units(), group=ps.get_fsdp_group() if world > 1 else False, device=dev,
                        param_dtype=param_dtype, **extra,
                        opt=opt, grad_accum_steps=accum, no_recompute=("lm_head",) if kind == "vlm" else ())
    std = getattr(getattr(model, "config", None), "init_std", 0.02)
    engine.materialize(stable_init_fn(std, args.seed))
    warm = args.lr_warmup_fraction or 0.0
    sched = LRSchedule(lr=args.lr, train_iters=args.train_iters, lr_decay_style=args.lr_decay_style,
                       lr_warmup_ratio=warm, lr_warmup_steps=int(getattr(args, "lr_warmup_iters", 0) or 0),
                       lr_min=args.min_lr or 0.0)
    loss_type = "per_token_loss" if args.calculate_per_token_loss else "default"
    cfg = TrainConfig(train_iters=args.train_iters, micro_batch_size=args.micro_batch_size,
                      gradient_accumulation_steps=accum, global_batch_size=args.global_batch_size,
                      log_interval=args.log_interval, save_interval=args.save_interval or 0,
                      exit_interval=int(args.exit_interval or 0), exit_duration_in_mins=float(args.exit_duration_in_mins or 0),
                      log_tps=bool(args.log_tps))
    ck = None
    if args.save or args.load:
        from ..checkpoint.sharded import DistributedCheckpointer
        ck = DistributedCheckpointer(args.save, args.load, no_save_optim=args.no_save_optim, no_save_rng=args.no_save_rng)
    prof_cfg = args.mm.tool.get("profile", None) if hasattr(args.mm, "tool") else None
    prof = None
    if prof_cfg is not None and getattr(prof_cfg, "enable", False):
        sp = prof_cfg.static_param
        prof = Profiler(True, getattr(prof_cfg, "ranks", [0]), sp.start_step, sp.end_step, sp.save_path)
    slog = None
    if getattr(args, "tensorboard_dir", None) or getattr(args, "wandb_project", None):
        from .logging import ScalarLog
        slog = ScalarLog(args.tensorboard_dir, getattr(args, "wandb_project", None), getattr(args, "wandb_save_dir", None),
                         getattr(args, "wandb_exp_name", None), int(getattr(args, "tensorboard_log_interval", None) or 1))
    ema = None
    if args.use_ema:
        from .ema import ShardedEMA
        ema = ShardedEMA(engine, decay=float(getattr(args, "ema_decay", None) or 0.9999), warmup=False)
    if getattr(args, "encoder_dp_balance", False) and kind == "vlm" and ps.get_dp_world_size() > 1:
        from ..parallel.data_balance import EncoderBalance
        model.encoder_balance = EncoderBalance(ps.group("dp"))
    te = TrainEngine(model, engine, build_loss(loss_type, ps.group("dp"), ps.get_dp_world_size()), sched, cfg,
                     data_iter=None, checkpointer=ck, profiler=prof,
                     dp_group=ps.group("dp"), dp_world=ps.get_dp_world_size(), device=dev, ema=ema, scalar_log=slog)
    if ck and args.load:
        te.load(load_optim=not args.no_load_optim, load_rng=not args.no_load_rng)
    # the sampler continues after the samples a resumed run has already consumed
    te.data_iter = datasets_provider(kind, args, model, ps, consumed_samples=te.consumed_train_samples)
    print_rank0(f"> parallel: {ps.describe()} | parameters: {engine.param_count() / 1e6:.1f} M")
    hist = te.train()
    if dist.is_initialized():
        dist.barrier()
    return hist
