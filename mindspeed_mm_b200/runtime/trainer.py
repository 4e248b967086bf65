"""Config-driven trainer for the native YAML schema.

    torchrun --nproc-per-node N -m mindspeed_mm_b200.runtime.trainer config.yaml [a.b.c=value ...]

Order of construction (reference: mindspeed_mm/fsdp/train/trainer.py:140-477): distributed init and seeds ->
plugins -> parallel state -> model on the meta device (+ freeze, LoRA) -> sharding engine (materialise /
load weights) -> optimizer hyper-parameters and LR schedule -> dataset, sampler, dataloader (optional
preloader) -> checkpointers -> profiler / memory profiler / watchdog -> ``TrainEngine.train()``.
"""
from __future__ import annotations

import json
import os
import random
import sys
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..api import init_distributed, stable_init_fn
from ..checkpoint import hf as hfio
from ..checkpoint.sharded import DistributedCheckpointer
from ..config.native import Arguments, load_config, match_modules
from ..config.tree import get_dtype
from ..models import registry
from ..parallel.fsdp import FSDPEngine, OptimConfig
from ..parallel.state import init_parallel_state
from .logging import print_rank0
from .loss import build_loss
from .lr_scheduler import LRSchedule
from .tools import MemoryProfiler, Profiler, Watchdog
from .train_engine import NativeKernelTimeout, TrainConfig, TrainEngine


def set_seed(seed: int, deterministic: bool = False) -> None:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")


class Trainer:
    def __init__(self, args: Arguments, device: Optional[str] = None):
        self.args = args
        t = args.training
        self.device, self.rank, self.world = init_distributed(device)
        set_seed(t.seed, t.use_deter_comp or t.enable_full_determinism)
        registry.import_plugin(t.plugin)
        registry._ensure_builtin()
        self.ps = init_parallel_state(world_size=self.world, device_type=self.device.type, **args.parallel.state_kwargs())
        self.model = self.build_model()
        self.engine = self.build_engine()
        if hasattr(self.model, "attach"):            # wrapped third-party classes: their sub-module calls go through the engine
            self.model.attach(self.engine, materialize=False)
        self.load_weights()
        self.schedule = LRSchedule(lr=t.lr, train_iters=t.train_iters, lr_decay_style=t.lr_decay_style,
                                   lr_warmup_ratio=t.lr_warmup_ratio, lr_min=t.lr_min, lr_start=t.lr_start,
                                   lr_decay_ratio=t.lr_decay_ratio)
        self.data_iter, self.val_iter_fn = self.build_data()
        self.checkpointer = self.build_checkpointer()
        cfg = TrainConfig(train_iters=t.train_iters, micro_batch_size=t.micro_batch_size,
                          gradient_accumulation_steps=t.gradient_accumulation_steps or 1,
                          global_batch_size=t.global_batch_size, log_interval=t.log_interval,
                          save_interval=t.save_interval, val_interval=t.val_interval, exit_interval=t.exit_interval,
                          exit_duration_in_mins=t.exit_duration_in_mins)
        self.train_engine = TrainEngine(
            self.model, self.engine, build_loss(args.features.loss_cfg.loss_type or "default", self.ps.group("dp"),
                                                self.ps.get_dp_world_size()),
            self.schedule, cfg, data_iter=self.data_iter, val_iter_fn=self.val_iter_fn, checkpointer=self.checkpointer,
            profiler=Profiler.from_config(args.tools.profile),
            memory_profiler=MemoryProfiler(**args.tools.memory_profile.model_dump()),
            watchdog=Watchdog(t.watchdog_timeout_s).start() if t.watchdog_timeout_s else None,
            dp_group=self.ps.group("dp"), dp_world=self.ps.get_dp_world_size(), device=self.device,
            ema=self.build_ema(), scalar_log=self.build_scalar_log())
        if self.checkpointer and t.load and t.load_format != "hf" and not hfio.is_hf_checkpoint(t.load):
            self.train_engine.load(load_optim=not t.no_load_optim, load_rng=not t.no_load_rng)

    # ------------------------------------------------------------------------------------------
    def build_model(self):
        m = self.args.model
        cls = registry.model_register.get(m.model_id)
        if getattr(cls, "hf_fallback", False) and m.model_name_or_path and \
                os.path.exists(os.path.join(m.model_name_or_path, "config.json")):
            # a zoo id that is a switch setting of the composable model, pointed at a real checkpoint: run the architecture
            # the checkpoint names (stock transformers class, this package's kernels and sharding engine)
            cls = registry.model_register.get("hf_auto")
        cfg = self._model_config(cls, m)
        text = getattr(cfg, "text", None)
        if text is not None and hasattr(text, "ep_dispatcher"):
            d = self.args.parallel.ep_plan.dispatcher
            text.ep_dispatcher = "p2p" if d in ("mc2", "fused") else d
        with torch.device("meta"):
            model = cls(cfg)
        names = [n for n, _ in model.named_modules()]
        for n in match_modules(m.freeze, names):
            for p in dict(model.named_modules())[n].parameters():
                p.requires_grad_(False)
        if self.args.training.lora.enable:
            from ..tasks.lora import apply_lora
            apply_lora(model, self.args.training.lora)
        return model

    def _model_config(self, cls, m):
        """``model_name_or_path/config.json`` (Hugging Face) describes the architecture when it exists; an inline
        ``model.config`` block then only overrides single fields (its ``preset`` is ignored).  Without a checkpoint
        directory the inline block, or a bare ``preset``, builds the config."""
        extra = m.model_extra or {}
        inline = extra.get("config")
        if m.model_name_or_path and os.path.exists(os.path.join(m.model_name_or_path, "config.json")):
            with open(os.path.join(m.model_name_or_path, "config.json")) as f:
                cfg = _config_from_hf(cls, json.load(f))
            return _config_from_dict(cls, {k: v for k, v in (inline or {}).items() if k != "preset"}, base=cfg)
        if inline is not None:
            return _config_from_dict(cls, inline)
        return _config_from_dict(cls, {"preset": extra.get("preset", "tiny")})

    def build_engine(self) -> FSDPEngine:
        a, t, plan = self.args, self.args.training, self.args.parallel.fsdp_plan
        opt = OptimConfig(lr=t.lr, betas=(t.adam_beta1, t.adam_beta2), eps=t.adam_eps, weight_decay=t.weight_decay,
                          clip_grad=t.clip_grad, clip_grad_ema_decay=t.clip_grad_ema_decay,
                          kind="muon" if t.optimizer == "muon" else "adamw",
                          muon_momentum=t.muon_momentum, ns_steps=t.ns_steps, matched_adamw_rms=t.matched_adamw_rms,
                          lr_scaling=tuple((p.match, p.scale) for p in (t.lr_scaling_plan or ())))
        if t.no_decay_params or t.no_decay_modules:
            keys = tuple(t.no_decay_params) + tuple(t.no_decay_modules)
            opt.no_decay = lambda n, p: p.dim() < 2 or any(k in n for k in keys)
        units = self.model.fsdp_units()
        recompute = a.features.recompute or a.parallel.recompute
        group = self.ps.get_fsdp_group() if self.world > 1 else False
        common = dict(device=self.device, param_dtype=get_dtype(plan.param_dtype or "bf16")
                      if self.device.type == "cuda" else torch.float32,
                      reduce_dtype=get_dtype(plan.reduce_dtype or "fp32"), opt=opt,
                      grad_accum_steps=t.gradient_accumulation_steps or 1)
        prefetch = max(plan.num_to_forward_prefetch or 0, plan.num_to_backward_prefetch or 0)
        # hybrid sharding: shard inside dp_shard(_cp), replicate over dp_replicate
        rep = self.ps.group("dp_replicate") if self.world > 1 and self.ps.size("dp_replicate") > 1 else None
        common.update(replicate_group=rep, offload_optimizer=bool(plan.cpu_offload or t.optimizer == "adamw_swap"))
        expert_units = self.model.expert_units() if hasattr(self.model, "expert_units") else []
        if not expert_units:
            eng = FSDPEngine(units, group=group, recompute=recompute, prefetch=prefetch, comm=plan.comm, **common)
            self._apply_plan(eng, units)
            return eng
        # MoE: dense parameters over the FSDP group; expert parameters over the expert-FSDP group (size 1 when
        # ep == ranks per stage), their gradients divided by the full data-parallel size.
        from ..parallel.fsdp import EngineMux
        ex = [p for _, m in expert_units for p in m.parameters()]
        dense = FSDPEngine(units, group=group, recompute=recompute, prefetch=prefetch, comm=plan.comm, exclude_params=ex,
                           **common)
        self._apply_plan(dense, units)
        common.update(replicate_group=None)
        eg = self.ps.group("efsdp") if self.ps.size("efsdp") > 1 else False
        expert = FSDPEngine(expert_units, group=eg, grad_divide=self.ps.get_dp_world_size(), no_recompute=(),
                            comm="nccl", **common)
        return EngineMux(dense, expert, ep_group=self.ps.group("ep") if self.ps.size("ep") > 1 else None)

    def build_scalar_log(self):
        tl = self.args.tools
        if not (tl.tensorboard_dir or tl.wandb_project):
            return None
        from .logging import ScalarLog
        return ScalarLog(tl.tensorboard_dir, tl.wandb_project, tl.wandb_save_dir, tl.wandb_exp_name, tl.tensorboard_log_interval)

    def build_ema(self):
        """``training.use_ema``: a moving average of the fp32 master shards, kept per rank and checkpointed with it."""
        t = self.args.training
        if not t.use_ema:
            return None
        from .ema import ShardedEMA
        return ShardedEMA(self.engine, decay=t.ema_decay, warmup=False)

    def hf_ops(self):
        """Hugging Face <-> internal name / layout map of the model, when it has one."""
        ops = getattr(self.model, "hf_ops", None)
        if ops is None and self.args.model.model_id == "qwen2_5vl":
            ops = hfio.qwen25vl_ops(self.model.config)
        return ops() if callable(ops) else ops

    def build_checkpointer(self):
        """Training checkpoints: torch DCP (``iter_XXXXXXX/`` with Hugging Face parameter names, the layout of the
        reference's native trainer) for data-parallel sharding; per-rank shard files (``save_format: sharded``, and always
        under expert / tensor / pipeline parallelism, where ranks hold different parameters).  A load directory is read
        in the format it was written in."""
        t = self.args.training
        if not (t.save or t.load):
            return None
        load = t.load if t.load_format != "hf" else None
        from ..parallel.fsdp import EngineMux
        plain = not isinstance(self.engine, EngineMux) and self.ps.size("tp") == 1 and self.ps.size("pp") == 1
        fmt = "dcp" if (plain and t.save_format in ("dcp", "auto", "hf")) else "sharded"
        if load and os.path.isdir(load):
            from ..checkpoint.sharded import read_tracker, iter_dir
            tag = open(os.path.join(load, "latest_checkpointed_iteration.txt")).read().strip() \
                if os.path.exists(os.path.join(load, "latest_checkpointed_iteration.txt")) else ""
            sub = os.path.join(load, "release") if tag == "release" else (iter_dir(load, int(tag)) if tag else load)
            if os.path.isdir(sub):
                fmt = "dcp" if os.path.exists(os.path.join(sub, ".metadata")) else "sharded"
        if fmt == "dcp":
            from ..checkpoint.dcp import TorchDCPCheckpointer
            return TorchDCPCheckpointer(t.save, load, t.save_async, t.no_save_optim, t.no_save_rng, ops=self.hf_ops())
        return DistributedCheckpointer(t.save, load, t.save_async, t.no_save_optim, t.no_save_rng)

    def _apply_plan(self, eng: FSDPEngine, units) -> None:
        """``fsdp_plan`` and memory features of the native schema, applied to the sharding engine."""
        a, plan, feat = self.args, self.args.parallel.fsdp_plan, self.args.features
        names = [n for n, _ in units]
        mod_names = [n for n, _ in self.model.named_modules()]
        wanted = None
        if plan.apply_modules:
            hit = set(match_modules(plan.apply_modules, names))
            # a pattern may name a parent of several units ("model.visual") or the model itself: those add nothing
            if hit:
                wanted = hit
        eng.select_units(wanted, reshard_after_forward=plan.reshard_after_forward)
        for n in match_modules(plan.ignored_modules, mod_names):
            m = dict(self.model.named_modules())[n]
            if any(p.requires_grad for p in m.parameters()):
                raise ValueError(f"fsdp_plan.ignored_modules: '{n}' has trainable parameters; the sharding engine owns every "
                                 f"trainable parameter (freeze the module with model.freeze to leave it out of training)")
        if feat.enable_activation_offload:
            from .features import ActivationOffload
            pats = feat.activation_offload_plan.apply_modules or []
            eng.set_activation_offload(ActivationOffload(self.device), match_modules(pats, names) if pats else names)
        if feat.enable_chunk_mbs and feat.chunkmbs_plan.apply_modules:
            from .features import chunk_mbs
            cp = feat.chunkmbs_plan
            table = dict(self.model.named_modules())
            for n in match_modules(cp.apply_modules, mod_names):
                table[n].forward = chunk_mbs(table[n].forward, cp.chunk_mbs, cp.batch_dim, tuple(cp.chunk_arg_indexs),
                                             tuple(cp.chunk_kwarg_names))
        if feat.enable_ep_balance:             # expert modules duplicate their hottest experts onto idle ranks per call
            for m in self.model.modules():
                if hasattr(m, "ep_balance_max_dup"):
                    m.ep_balance_max_dup = int(feat.ep_balance_plan.max_dup_experts_num)

    def load_weights(self):
        t = self.args.training
        std = getattr(getattr(self.model, "config", None), "init_std", 0.02)
        self.engine.materialize(stable_init_fn(std, t.seed))
        path = t.load or self.args.model.model_name_or_path
        fmt = t.load_format
        if path and (fmt == "hf" or (fmt == "auto" and hfio.is_hf_checkpoint(path))):
            ops = self.hf_ops()
            if ops is not None:
                hfio.load_hf_into_engine(self.engine, path, ops, strict=t.load_strict and not t.lora.enable)
        if t.lora.enable and t.lora.pretrained_lora_path:          # adapter files in PEFT's layout
            from safetensors.torch import load_file
            from ..tasks.lora import from_peft_state
            ad = from_peft_state(load_file(os.path.join(t.lora.pretrained_lora_path, "adapter_model.safetensors")), self.hf_ops())
            self.engine.load_full_params(lambda name, shape: ad[name].to(self.device) if name in ad else None)

    def build_data(self):
        from ..data import build_dataloader
        return build_dataloader(self.args, self.model, self.ps, self.device)

    def train(self):
        hist = self.train_engine.train()
        t = self.args.training
        if t.lora.enable and t.save and self.hf_ops() is not None:       # adapter-only files in PEFT's layout
            from ..tasks.lora import lora_state_dict, save_peft_adapter
            state = lora_state_dict(self.engine.named_full_params())    # every rank takes part in the gathers
            if self.rank == 0:
                save_peft_adapter(state, self.hf_ops(), os.path.join(t.save, "lora_adapter"), t.lora,
                                  self.args.model.model_name_or_path or "")
        ops = self.hf_ops() if (t.save and t.save_format == "hf" and not t.lora.enable) else None
        if ops is not None:
            if self.train_engine.ema is not None:          # export the averaged weights, then put the live ones back
                self.train_engine.ema.swap()
            hfio.save_engine_as_hf(self.engine, os.path.join(t.save, "hf"), ops,
                                   get_dtype(t.save_ckpt_dtype) if t.save_ckpt_dtype else None,
                                   self.args.model.model_name_or_path, self.rank)
            if self.train_engine.ema is not None:
                self.train_engine.ema.swap()
        if self.checkpointer:
            self.checkpointer.wait()
        return hist


def _config_from_dict(cls, d: dict, base=None):
    cfg_cls = _config_class(cls)
    preset = d.get("preset")
    cfg = base if base is not None else (getattr(cfg_cls, preset)() if preset and hasattr(cfg_cls, preset) else cfg_cls())
    for k, v in d.items():
        if k == "preset":
            continue
        if isinstance(v, dict) and hasattr(cfg, k):
            sub = getattr(cfg, k)
            for kk, vv in v.items():
                setattr(sub, kk, tuple(vv) if isinstance(vv, list) else vv)
        elif hasattr(cfg, k):
            setattr(cfg, k, tuple(v) if isinstance(v, list) else v)
    return cfg


def _config_from_hf(cls, hf: dict):
    cfg_cls = _config_class(cls)
    if hasattr(cfg_cls, "from_hf"):
        return cfg_cls.from_hf(hf)
    return cfg_cls()


def _config_class(cls):
    import inspect
    if getattr(cls, "config_class", None) is not None:
        return cls.config_class
    sig = inspect.signature(cls.__init__)
    ann = list(sig.parameters.values())[1].annotation
    if isinstance(ann, str):
        mod = sys.modules[cls.__module__]
        ann = getattr(mod, ann)
    return ann


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit("usage: trainer.py config.yaml [key=value ...]")
    args = load_config(argv[0], argv[1:])
    tr = Trainer(args)
    try:
        tr.train()
    except NativeKernelTimeout as e:
        print(f"[rank {dist.get_rank() if dist.is_initialized() else 0}] {e}", file=sys.stderr, flush=True)
        os._exit(e.exit_code)          # peers may be gone: no collective shutdown
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
