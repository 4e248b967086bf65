"""Public, programmatic entry points (what ``bench.py`` and user scripts call).

``build_vlm_trainer`` assembles the pieces the YAML-driven ``Trainer`` assembles from a config file:
process group + parallel state, the model on the meta device, the sharding engine (which owns the
optimizer), loss, LR schedule and the ``TrainEngine`` loop.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel
from .parallel.fsdp import FSDPEngine, OptimConfig
from .parallel.state import get_parallel_state, init_parallel_state
from .runtime.loss import build_loss
from .runtime.lr_scheduler import LRSchedule
from .runtime.train_engine import TrainConfig, TrainEngine


def init_distributed(device: Optional[str] = None, timeout_s: int = 600):
    """One process per GPU; reads RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment."""
    import datetime
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if device == "cuda":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        backend = "nccl" if dev.type == "cuda" else "gloo"
        kw = dict(device_id=dev) if dev.type == "cuda" else {}
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return dev, (dist.get_rank() if dist.is_initialized() else 0), world


def default_init_fn(std: float = 0.02, seed: int = 0):
    """Random init executed on the unit's device: N(0, std) for matrices, 1 for norm weights, 0 for biases.
    Seeded per unit name so every rank (and every world size) draws the same full tensor."""
    def init(name: str, module: nn.Module):
        for n, p in module.named_parameters():
            g = torch.Generator(device=p.device).manual_seed((hash((name, n)) & 0x7FFFFFFF) ^ seed)
            if p.dim() >= 2:
                p.data.normal_(0.0, std, generator=g)
            elif n.endswith("bias"):
                p.data.zero_()
            else:
                p.data.fill_(1.0)
        for m in module.modules():
            if hasattr(m, "post_init"):
                m.post_init()
    return init


@dataclass
class VLMTrainerSpec:
    model: Qwen25VLConfig
    lr: float = 1e-5
    weight_decay: float = 0.0
    clip_grad: float = 0.0
    train_iters: int = 10000
    lr_decay_style: str = "cosine"
    lr_warmup_ratio: float = 0.1
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    param_dtype: torch.dtype = torch.bfloat16
    reduce_dtype: torch.dtype = torch.float32
    recompute: object = True          # True / False / "auto" / int = number of decoder layers to recompute
    tokens_per_micro_batch: int = 8192   # used by recompute="auto" to size the activation budget
    patches_per_micro_batch: int = 8192  # vision patches per micro-batch, same purpose
    activation_reserve_gb: float = 20.0  # memory kept free for workspaces when recompute="auto"
    loss_type: str = "default"
    seed: int = 0
    comm: str = "auto"
    freeze_vision: bool = False
    log_interval: int = 1
    shard_size: Optional[int] = None     # < number of data ranks: hybrid sharding (shard inside, replicate across)
    offload_optimizer: bool = False      # fp32 master weights + Adam moments in pinned host memory
    optimizer: str = "adamw"             # "muon": Newton-Schulz orthogonalised momentum for the 2-D hidden matrices
    lr_scaling: tuple = ()               # ((regex, multiplier), ...) on parameter names
    reshard_after_forward: bool = True


def build_vlm_trainer(spec: VLMTrainerSpec, device=None, data_iter=None, checkpointer=None) -> TrainEngine:
    dev, rank, world = init_distributed(None if device is None else str(device).split(":")[0])
    ps = init_parallel_state(world_size=world, device_type=dev.type,
                             fully_shard_parallel_size=spec.shard_size if spec.shard_size else "auto")
    with torch.device("meta"):
        model = Qwen25VLModel(spec.model)
    if spec.freeze_vision:
        for p in model.visual.parameters():
            p.requires_grad_(False)
    opt = OptimConfig(lr=spec.lr, weight_decay=spec.weight_decay, clip_grad=spec.clip_grad, kind=spec.optimizer,
                      lr_scaling=tuple(spec.lr_scaling))
    engine = FSDPEngine(model.fsdp_units(), group=ps.get_fsdp_group() if world > 1 else False, device=dev,
                        param_dtype=spec.param_dtype, reduce_dtype=spec.reduce_dtype, opt=opt,
                        recompute=spec.recompute is not False, grad_accum_steps=spec.gradient_accumulation_steps,
                        comm=spec.comm, offload_optimizer=spec.offload_optimizer,
                        replicate_group=ps.group("dp_replicate") if world > 1 and ps.size("dp_replicate") > 1 else None)
    engine.select_units(None, reshard_after_forward=spec.reshard_after_forward)
    # python's hash() of str is salted per process: use a stable digest instead
    engine.materialize(stable_init_fn(spec.model.init_std, spec.seed))
    if spec.recompute == "auto" or (isinstance(spec.recompute, int) and not isinstance(spec.recompute, bool)):
        plan_recompute(engine, spec, world)
    sched = LRSchedule(lr=spec.lr, train_iters=spec.train_iters, lr_decay_style=spec.lr_decay_style,
                       lr_warmup_ratio=spec.lr_warmup_ratio)
    loss_fn = build_loss(spec.loss_type, ps.group("dp"), ps.get_dp_world_size())
    cfg = TrainConfig(train_iters=spec.train_iters, micro_batch_size=spec.micro_batch_size,
                      gradient_accumulation_steps=spec.gradient_accumulation_steps, log_interval=spec.log_interval)
    return TrainEngine(model, engine, loss_fn, sched, cfg, data_iter=data_iter, checkpointer=checkpointer,
                       dp_group=ps.group("dp"), dp_world=ps.get_dp_world_size(), device=dev)


def decoder_layer_activation_bytes(t, tokens: int) -> int:
    """Bytes autograd keeps for one decoder layer when it is not recomputed: the inputs of both norms and of the
    four GEMMs, the rotated q/k, the attention output and the SwiGLU input (bf16), plus fp32 row statistics."""
    qkv = (t.num_attention_heads + 2 * t.num_key_value_heads) * t.head_dim
    rot = (t.num_attention_heads + t.num_key_value_heads) * t.head_dim
    per_token = 2 * (5 * t.hidden_size + qkv + rot + 3 * t.intermediate_size) + 4 * (2 + t.num_attention_heads)
    return per_token * tokens


def vision_block_activation_bytes(v, patches: int) -> int:
    inter = -(-v.intermediate_size // 64) * 64
    return (2 * (5 * v.hidden_size + 3 * v.hidden_size + 2 * v.hidden_size + 3 * inter) + 4 * (2 + v.num_heads)) * patches


def plan_recompute(engine: FSDPEngine, spec: VLMTrainerSpec, world: int) -> int:
    """Keep the autograd graph of as many decoder layers as the free device memory allows (the last layers first:
    their backward runs first) and recompute the rest.  Returns the number of layers left on recompute.  All ranks
    take the minimum so that they run the same plan."""
    layers = [u for u in engine.units if u.name.startswith("layers.")]
    if isinstance(spec.recompute, int) and not isinstance(spec.recompute, bool):
        keep = max(0, len(layers) - spec.recompute)
    elif engine.device.type == "cuda":
        free, _ = torch.cuda.mem_get_info(engine.device)
        per_layer = decoder_layer_activation_bytes(spec.model.text, spec.tokens_per_micro_batch) * 1.1
        # a layer that keeps its graph also keeps its gathered bf16 weights and gradients until its update
        per_layer += 0 if world == 1 else 4 * sum(g.padded for g in layers[0].groups)
        keep = int(max(0.0, free - spec.activation_reserve_gb * 2 ** 30) // per_layer)
        if world > 1:
            k = torch.tensor([keep], device=engine.device)
            dist.all_reduce(k, op=dist.ReduceOp.MIN)
            keep = int(k.item())
    else:
        keep = 0
    keep = min(keep, len(layers))
    for u in layers[len(layers) - keep:]:
        u.recompute = False
    engine.recompute_plan = {"decoder_layers": len(layers), "recomputed": len(layers) - keep}
    blocks = [u for u in engine.units if u.name.startswith("visual.blocks.") and u.trainable]
    engine.recompute_plan.update(vision_blocks=len(blocks), vision_recomputed=len(blocks))
    if spec.recompute == "auto" and keep == len(layers) and blocks and engine.device.type == "cuda":
        left = free - spec.activation_reserve_gb * 2 ** 30 - keep * per_layer
        per_block = vision_block_activation_bytes(spec.model.vision, spec.patches_per_micro_batch) * 1.1
        per_block += 0 if world == 1 else 4 * sum(g.padded for g in blocks[0].groups)
        kb = int(max(0.0, left) // per_block)
        if world > 1:
            k = torch.tensor([kb], device=engine.device)
            dist.all_reduce(k, op=dist.ReduceOp.MIN)
            kb = int(k.item())
        kb = min(kb, len(blocks))
        for u in blocks[len(blocks) - kb:]:
            u.recompute = False
        engine.recompute_plan["vision_recomputed"] = len(blocks) - kb
    return len(layers) - keep


def wan_block_activation_bytes(c, tokens_local: int) -> int:
    """Bytes autograd keeps for one Wan DiT block (self-attention incl. the Ulysses-exchanged q/k/v/o, cross-attention,
    GELU FFN) when it is not recomputed."""
    return 2 * (23 * c.hidden_size + 2 * c.ffn_dim) * tokens_local


def plan_recompute_units(engine: FSDPEngine, prefix: str, per_unit_bytes: float, reserve_gb: float = 20.0) -> dict:
    """Generic form of :func:`plan_recompute`: keep the graph of as many ``prefix*`` units (last ones first) as the
    free device memory allows."""
    units = [u for u in engine.units if u.name.startswith(prefix)]
    keep = 0
    if engine.device.type == "cuda" and units:
        free, _ = torch.cuda.mem_get_info(engine.device)
        per = per_unit_bytes * 1.1 + (0 if engine.world == 1 else 4 * sum(g.padded for g in units[0].groups))
        keep = int(max(0.0, free - reserve_gb * 2 ** 30) // per)
        if engine.world > 1:
            k = torch.tensor([keep], device=engine.device)
            dist.all_reduce(k, op=dist.ReduceOp.MIN, group=engine.group)
            keep = int(k.item())
    keep = min(keep, len(units))
    for u in units[len(units) - keep:]:
        u.recompute = False
    engine.recompute_plan = {"units": len(units), "recomputed": len(units) - keep}
    return engine.recompute_plan


def stable_init_fn(std: float = 0.02, seed: int = 0):
    import zlib

    def init(name: str, module: nn.Module):
        for n, p in module.named_parameters():
            s = (zlib.crc32(f"{name}.{n}".encode()) ^ seed) & 0x7FFFFFFF
            if p.dim() >= 2:
                g = torch.Generator(device=p.device).manual_seed(s)
                p.data.normal_(0.0, std, generator=g)
            elif n.endswith("bias"):
                p.data.zero_()
            else:
                p.data.fill_(1.0)
        for m in module.modules():
            if hasattr(m, "post_init"):
                m.post_init()
    return init
