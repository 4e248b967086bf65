"""Legacy launch schema: Megatron-style flags + ``--mm-model / --mm-data / --mm-tool`` JSON or YAML files.

``parse_legacy_args(argv)`` accepts the flag vocabulary the reference's shell recipes pass
(examples/qwen2.5vl/finetune_qwen2_5_vl_7b.sh:59-111, examples/wan2.1/14b/t2v/pretrain.sh) - known flags are
typed, unknown ``--flags`` are kept (as strings / booleans) so that a recipe never dies on an option that
only matters to another backend - and attaches ``args.mm.{model,data,tool}`` attribute trees
(mindspeed_mm/configs/config.py:67-140).  A first positional ``*.yaml`` switches to the single-file schema
(``gpt_args`` / ``lora_args`` flattened to flags, ``MM_TOOL_PATH``; mindspeed_mm/configs/read_yaml_config.py:9-78).
"""
from __future__ import annotations

import argparse
import json
import os
from types import SimpleNamespace
from typing import Any, Dict, List, Optional, Sequence

import yaml

from .security import check_args_paths
from .tree import ConfigNode


class MMConfig:
    """``MMConfig({"model": path, "data": path, "tool": path})`` -> ``.model/.data/.tool`` trees.
    A ``.yaml`` path contributes its top-level entry of the same name."""

    def __init__(self, files: Dict[str, str]):
        errors = []
        for name, path in files.items():
            if not path:
                continue
            try:
                real = os.path.realpath(path)
                if real.endswith(".json"):
                    with open(real) as f:
                        d = json.load(f)
                elif real.endswith((".yaml", ".yml")):
                    with open(real) as f:
                        d = yaml.safe_load(f)[name]
                else:
                    raise ValueError("config files must be .json or .yaml")
                setattr(self, name, ConfigNode(d))
            except FileNotFoundError as e:
                errors.append(f"Warning: Config file not found: {path} - {e}")
            except (json.JSONDecodeError, yaml.YAMLError) as e:
                errors.append(f"Error: Invalid format in {path}: {e}")
            except Exception as e:  # noqa: BLE001
                errors.append(f"Error: Unexpected error loading {path}: {e}")
        if errors:
            raise RuntimeError("One or more config files failed to load:\n" + "\n".join(errors))


def yaml_to_argv(config_path: str) -> List[str]:
    """Flatten ``gpt_args`` (+ ``lora_args``) of a single-file recipe into Megatron flags."""
    with open(config_path) as f:
        cfg = yaml.safe_load(f)
    if "gpt_args" not in cfg:
        raise KeyError("The required keyword 'gpt_args' is missing from the configuration file.")
    if "MM_TOOL_PATH" not in cfg:
        raise KeyError("The required keyword 'MM_TOOL_PATH' is missing from the configuration file.")
    flat: Dict[str, Any] = {}

    def walk(d):
        for k, v in d.items():
            if isinstance(v, dict):
                walk(v)
            else:
                flat[k.replace("_", "-")] = v

    walk(cfg["gpt_args"])
    if "lora_args" in cfg:
        walk(cfg["lora_args"])
    argv: List[str] = []
    for k, v in flat.items():
        if isinstance(v, bool):
            if v:
                argv.append(f"--{k}")
        elif isinstance(v, list):
            for x in v:
                argv += [f"--{k}", str(x)]
        elif v is not None:
            argv += [f"--{k}", str(v)]
    argv += ["--mm-data", config_path, "--mm-model", config_path, "--mm-tool", cfg["MM_TOOL_PATH"]]
    return argv


_INT = ["tensor-model-parallel-size", "pipeline-model-parallel-size", "context-parallel-size",
        "expert-model-parallel-size", "micro-batch-size", "global-batch-size", "seq-length", "vocab-size",
        "train-iters", "log-interval", "save-interval", "eval-interval", "eval-iters", "num-workers", "seed",
        "num-layers", "hidden-size", "num-attention-heads", "max-position-embeddings", "lr-warmup-iters",
        "exit-interval", "ulysses-degree-in-cp", "virtual-pipeline-model-parallel-size", "recompute-num-layers",
        "make-vocab-size-divisible-by", "distributed-timeout-minutes", "num-layers-per-virtual-pipeline-stage",
        "tensorboard-log-interval"]
_FLOAT = ["ema-decay", "lr", "min-lr", "weight-decay", "clip-grad", "adam-beta1", "adam-beta2", "adam-eps", "lr-warmup-fraction",
          "init-method-std", "exit-duration-in-mins", "attention-dropout", "hidden-dropout"]
_STR = ["lr-decay-style", "tokenizer-type", "load", "save", "ckpt-format", "distributed-backend", "mm-data",
        "mm-model", "mm-tool", "context-parallel-algo", "fsdp2-config-path", "normalization", "recompute-granularity",
        "recompute-method", "position-embedding-type", "optimizer", "tensorboard-dir", "layerzero-config",
        "load-base-model", "dataloader-type", "attention-mask-type", "wandb-project", "wandb-exp-name", "wandb-save-dir"]
_BOOL = ["bf16", "fp16", "use-mcore-models", "use-flash-attn", "use-distributed-optimizer", "use-torch-fsdp2",
         "sequence-parallel", "swiglu", "use-fused-swiglu", "use-fused-rmsnorm", "use-fused-rotary-pos-emb",
         "no-load-optim", "no-load-rng", "no-save-optim", "no-save-rng", "variable-seq-lengths", "log-tps",
         "untie-embeddings-and-output-weights", "no-gradient-accumulation-fusion", "use-cpu-initialization",
         "init-model-with-meta-device", "no-initialization", "overlap-grad-reduce", "overlap-param-gather",
         "calculate-per-token-loss", "calculate-per-sample-loss", "layerzero", "use-deter-comp", "no-masked-softmax-fusion",
         "disable-bias-linear", "group-query-attention", "recompute-skip-core-attention", "use-ema", "no-bias-swiglu-fusion",
         "encoder-dp-balance", "use-data-balance", "hetero-parallel"]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(allow_abbrev=False, add_help=False)
    for n in _INT:
        p.add_argument(f"--{n}", type=int, default=None)
    for n in _FLOAT:
        p.add_argument(f"--{n}", type=float, default=None)
    for n in _STR:
        p.add_argument(f"--{n}", type=str, default=None)
    for n in _BOOL:
        p.add_argument(f"--{n}", action="store_true", default=False)
    return p


DEFAULTS = dict(tensor_model_parallel_size=1, pipeline_model_parallel_size=1, context_parallel_size=1,
                expert_model_parallel_size=1, micro_batch_size=1, train_iters=10, log_interval=1, lr=1e-5,
                min_lr=0.0, weight_decay=0.0, clip_grad=1.0, adam_beta1=0.9, adam_beta2=0.999, adam_eps=1e-8,
                lr_decay_style="cosine", lr_warmup_fraction=0.0, seed=1234, save_interval=0, eval_interval=0,
                distributed_backend="nccl", ckpt_format="torch", context_parallel_algo="ulysses_cp_algo",
                mm_model="", mm_data="", mm_tool="", num_workers=0)


def parse_legacy_args(argv: Optional[Sequence[str]] = None, check_paths: bool = True) -> SimpleNamespace:
    import sys
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0].endswith((".yaml", ".yml")):
        argv = yaml_to_argv(argv[0]) + argv[1:]
    known, unknown = build_parser().parse_known_args(argv)
    args = SimpleNamespace(**{k: v for k, v in vars(known).items()})
    for k, v in DEFAULTS.items():
        if getattr(args, k, None) is None:
            setattr(args, k, v)
    # keep unknown flags: "--flag value" or bare "--flag"
    extra: Dict[str, Any] = {}
    i = 0
    while i < len(unknown):
        tok = unknown[i]
        if tok.startswith("--"):
            key = tok[2:].replace("-", "_")
            if "=" in key:
                key, val = key.split("=", 1)
                extra[key] = val
            elif i + 1 < len(unknown) and not unknown[i + 1].startswith("--"):
                extra[key] = unknown[i + 1]
                i += 1
            else:
                extra[key] = True
        i += 1
    for k, v in extra.items():
        if not hasattr(args, k):
            setattr(args, k, v)
    args.unknown_args = extra
    args.global_batch_size_given = args.global_batch_size is not None
    if args.global_batch_size is None:
        args.global_batch_size = args.micro_batch_size
    merge_mm_args(args)
    if check_paths:
        args.path_warnings = check_args_paths(args, warn=lambda *_: None)
    return args


def validate_args(args, world_size: int) -> SimpleNamespace:
    """Consistency checks and derived sizes of the Megatron-style flag set, done once before anything is built
    (the reference replaces Megatron's ``validate_args`` with its own: mindspeed_mm/patchs/validate_args_patch.py:33).
    Raises ``ValueError`` naming the flags at fault; returns the derived values (``data_parallel_size``,
    ``num_micro_batches``, ``ulysses_size``, ``ring_size``, ``sequence_parallel``, ``params_dtype``)."""
    tp, pp, cp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size, args.context_parallel_size
    ep = args.expert_model_parallel_size
    problems: List[str] = []
    for name, v in (("tensor-model-parallel-size", tp), ("pipeline-model-parallel-size", pp), ("context-parallel-size", cp),
                    ("expert-model-parallel-size", ep), ("micro-batch-size", args.micro_batch_size)):
        if v is None or v < 1:
            problems.append(f"--{name} must be >= 1 (got {v})")
    if problems:
        raise ValueError("; ".join(problems))
    model_parallel = tp * pp * cp
    if world_size % model_parallel:
        raise ValueError(f"world size {world_size} is not divisible by tensor ({tp}) x pipeline ({pp}) x context ({cp}) parallel size")
    dp = world_size // model_parallel
    if ep > 1 and (dp * cp) % ep:
        problems.append(f"--expert-model-parallel-size {ep} must divide data x context parallel size {dp * cp}")
    gbs, mbs = args.global_batch_size or args.micro_batch_size * dp, args.micro_batch_size
    if gbs == mbs and not getattr(args, "global_batch_size_given", True):
        gbs = mbs * dp                   # the flag was not given: one micro-batch per data-parallel rank
    if gbs % (mbs * dp):
        problems.append(f"--global-batch-size {gbs} is not divisible by micro batch {mbs} x data parallel {dp}")
    if getattr(args, "bf16", False) and getattr(args, "fp16", False):
        problems.append("--bf16 and --fp16 are exclusive")
    if args.clip_grad is not None and args.clip_grad < 0:
        problems.append(f"--clip-grad must be >= 0 (got {args.clip_grad})")
    if args.min_lr is not None and args.lr is not None and args.min_lr > args.lr:
        problems.append(f"--min-lr {args.min_lr} is above --lr {args.lr}")
    if args.lr_warmup_fraction and getattr(args, "lr_warmup_iters", None):
        problems.append("--lr-warmup-fraction and --lr-warmup-iters are exclusive")
    vpp = getattr(args, "virtual_pipeline_model_parallel_size", None)
    per_stage = getattr(args, "num_layers_per_virtual_pipeline_stage", None)
    if (vpp and vpp > 1 or per_stage) and pp < 2:
        problems.append("virtual pipeline stages need --pipeline-model-parallel-size >= 2")
    n_layers = getattr(args, "num_layers", None)
    if n_layers and n_layers % pp:
        problems.append(f"--num-layers {n_layers} is not divisible by the pipeline size {pp} (give per-stage layer lists in the model json)")
    if n_layers and per_stage and (n_layers // pp) % per_stage:
        problems.append(f"layers per pipeline stage {n_layers // pp} are not divisible by --num-layers-per-virtual-pipeline-stage {per_stage}")
    seq = getattr(args, "seq_length", None)
    uly = getattr(args, "ulysses_degree_in_cp", None)
    algo = args.context_parallel_algo
    if cp > 1:
        if algo == "hybrid_cp_algo":
            if not uly or cp % uly:
                problems.append(f"hybrid context parallel needs --ulysses-degree-in-cp dividing --context-parallel-size {cp} (got {uly})")
        elif algo not in ("ulysses_cp_algo", "megatron_cp_algo"):
            problems.append(f"unknown --context-parallel-algo {algo}")
        ring = cp if algo == "megatron_cp_algo" else (cp // uly if algo == "hybrid_cp_algo" and uly else 1)
        if seq and seq % (cp * (2 if ring > 1 else 1)):
            problems.append(f"--seq-length {seq} must be a multiple of {cp * (2 if ring > 1 else 1)} for context parallel {cp}"
                            + (" (zig-zag halves of the ring)" if ring > 1 else ""))
        heads = getattr(args, "num_attention_heads", None)
        u = cp // ring
        if heads and u > 1 and (heads // tp) % u:
            problems.append(f"Ulysses degree {u} must divide the attention heads per tensor-parallel rank ({heads // tp})")
    else:
        ring = 1
    sp = bool(getattr(args, "sequence_parallel", False))
    if sp and tp == 1:
        sp = False                       # as Megatron does: nothing to scatter over
    if sp and seq and seq % tp:
        problems.append(f"--sequence-parallel needs --seq-length {seq} divisible by the tensor-parallel size {tp}")
    rg, rm, rn = (getattr(args, k, None) for k in ("recompute_granularity", "recompute_method", "recompute_num_layers"))
    if rg not in (None, "full", "selective"):
        problems.append(f"--recompute-granularity must be full or selective (got {rg})")
    if rm is not None and rg != "full":
        problems.append("--recompute-method needs --recompute-granularity full")
    if rm not in (None, "uniform", "block"):
        problems.append(f"--recompute-method must be uniform or block (got {rm})")
    if rn is not None and rm is None:
        problems.append("--recompute-num-layers needs --recompute-method")
    if getattr(args, "use_torch_fsdp2", False) and (tp > 1 or pp > 1):
        problems.append("--use-torch-fsdp2 shards over the whole data-parallel group: tensor / pipeline parallel sizes must be 1")
    if getattr(args, "layerzero", False) and getattr(args, "use_torch_fsdp2", False):
        problems.append("--layerzero and --use-torch-fsdp2 are exclusive")
    if getattr(args, "calculate_per_token_loss", False) and getattr(args, "calculate_per_sample_loss", False):
        problems.append("--calculate-per-token-loss and --calculate-per-sample-loss are exclusive")
    if problems:
        raise ValueError("invalid arguments:\n  " + "\n  ".join(problems))
    return SimpleNamespace(data_parallel_size=dp, num_micro_batches=gbs // (mbs * dp), ring_size=ring, ulysses_size=cp // ring,
                           sequence_parallel=sp, params_dtype="bf16" if getattr(args, "bf16", False) else
                           ("fp16" if getattr(args, "fp16", False) else "fp32"))


def merge_mm_args(args) -> None:
    if not hasattr(args, "mm") or args.mm is None:
        args.mm = MMConfig({"model": args.mm_model, "data": args.mm_data, "tool": args.mm_tool})


def load_fsdp2_config(path: str) -> dict:
    """The separate sharding YAML of the Megatron-style FSDP2 recipes (``--use-torch-fsdp2 --fsdp2-config-path``; schema:
    mindspeed_mm/models/transformers/base_model.py:220-283).  Returns the keys the engine uses, normalised:
    ``sharding_size`` (int or None = all data ranks), ``param_dtype`` / ``reduce_dtype`` (torch dtypes or None),
    ``reshard_after_forward`` (bool), ``recompute_modules`` / ``sub_modules_to_wrap`` (lists of patterns, kept for
    reporting: the unit list comes from the model's ``fsdp_units()``), ``offload_to_cpu`` (bool)."""
    import torch
    import yaml
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    dt = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
          "fp32": torch.float32, "float32": torch.float32, None: None}
    size = raw.get("sharding_size")
    out = {
        "sharding_size": None if size in (None, "auto", -1) else int(size),
        "param_dtype": dt[raw.get("param_dtype")],
        "reduce_dtype": dt[raw.get("reduce_dtype")],
        "reshard_after_forward": bool(raw.get("reshard_after_forward", True)),
        "sub_modules_to_wrap": list(raw.get("sub_modules_to_wrap") or []),
        "recompute_modules": list(raw.get("recompute_modules") or []),
        "offload_to_cpu": bool(raw.get("offload_to_cpu", False)),
    }
    unknown = sorted(set(raw) - set(out) - {"ignored_modules", "num_to_forward_prefetch", "num_to_backward_prefetch",
                                           "output_dtype", "cast_forward_inputs"})
    out["unknown_keys"] = unknown
    return out


def load_layerzero_config(path: str) -> dict:
    """The LayerZero (FSDP1-style ZeRO-3) YAML of the reference's Wan / HunyuanVideo recipes (``--layerzero
    --layerzero-config``; mindspeed_mm/patchs/fsdp1_patches.py:121, examples/wan2.1/zero_config.yaml), normalised to the
    keys of ``load_fsdp2_config``: ``zero3_size`` is the shard group size (smaller than the data ranks = hybrid sharding),
    ``transformer_layers`` names the wrapped block classes (reported only: units come from the model's ``fsdp_units()``),
    ``forward_prefetch`` / ``backward_prefetch`` turn the engine's one-unit look-ahead on or off."""
    import torch
    import yaml
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    dt = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
          "fp32": torch.float32, "float32": torch.float32, None: None}
    size = raw.get("zero3_size")
    out = {
        "sharding_size": None if size in (None, "auto", -1) else int(size),
        "param_dtype": dt[raw.get("param_dtype")],
        "reduce_dtype": dt[raw.get("reduce_dtype")],
        "reshard_after_forward": True,
        "sub_modules_to_wrap": [str(c).rsplit(".", 1)[-1] for c in (raw.get("transformer_layers") or [])],
        "recompute_modules": [],
        "offload_to_cpu": bool(raw.get("offload_to_cpu", False)),
        "prefetch": 1 if (raw.get("forward_prefetch", True) or raw.get("backward_prefetch") not in (None, "None", False)) else 0,
    }
    known = {"zero3_size", "param_dtype", "reduce_dtype", "transformer_layers", "offload_to_cpu", "forward_prefetch",
             "backward_prefetch", "limit_all_gathers", "ignored_modules", "ckpt_layers", "use_orig_params"}
    out["unknown_keys"] = sorted(set(raw) - known)
    return out

