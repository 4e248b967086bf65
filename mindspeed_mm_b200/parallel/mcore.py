"""Megatron-style backend: tensor parallel x pipeline parallel x data parallel (with sequence parallelism).

The LLM of a VLM is built per (tp rank, pp stage): fused QKV and gate|up are column-parallel (heads / FFN
columns split), o_proj and down_proj row-parallel, embedding and head vocabulary-parallel, layers sliced over
pipeline stages by ``pipeline_num_layers`` (models/vlm_model.py:300-345 in the reference).  The vision tower runs
replicated on the first stage's tensor-parallel ranks (they see identical inputs, so their gradients agree), or, with
``--hetero-parallel``, data parallel over them: each rank encodes a share of the micro-batch's images and the
embeddings are all-gathered (``parallel/hetero.py``; the reference's per-module parallel plans,
mindspeed_mm/utils/hetero_parallel.py:22-315).
Parameters of a (tp, pp) rank are then sharded over the data-parallel group by the flat-buffer engine, i.e. the
"distributed optimizer" of the Megatron recipes is the same ZeRO engine as the FSDP backend, and the training
loop, log line and checkpointing are shared.  ``shard_full_state`` cuts a full (HF-layout internal) state dict into
the local tensors of any (tp, pp) coordinate, which is also what the offline converter writes to mp_rank files.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..models.qwen2_5_vl import (Embedding, LMHead, PatchMerger, Qwen25VLConfig, RMSNorm, TextConfig, VisionBlock,
                                 VisionPatchEmbed, VisionTransformer)
from .pp import PipelineSchedule, split_layers
from .tp import (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding, gather_sequence, scatter_sequence,
                 split_sequence, vocab_parallel_cross_entropy)


class TPDecoderLayer(nn.Module):
    def __init__(self, c: TextConfig, tp_group, sp: bool):
        super().__init__()
        tp = dist.get_world_size(tp_group) if tp_group is not None else 1
        if c.num_key_value_heads % tp:
            raise ValueError(f"num_key_value_heads {c.num_key_value_heads} must be divisible by tp {tp}")
        self.nq, self.nkv, self.hd = c.num_attention_heads // tp, c.num_key_value_heads // tp, c.head_dim
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.qkv_proj = ColumnParallelLinear(c.hidden_size, (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim,
                                             tp_group, bias=c.qkv_bias, sequence_parallel=sp)
        self.o_proj = RowParallelLinear(c.num_attention_heads * c.head_dim, c.hidden_size, tp_group, bias=False,
                                        sequence_parallel=sp)
        self.gate_up_proj = ColumnParallelLinear(c.hidden_size, 2 * c.intermediate_size, tp_group, bias=False,
                                                 sequence_parallel=sp)
        self.down_proj = RowParallelLinear(c.intermediate_size, c.hidden_size, tp_group, bias=False, sequence_parallel=sp)
        if sp and tp > 1:      # norm weights are replicated but each replica only sees its sequence slice
            self.input_layernorm.weight._tp_sum_group = tp_group
            self.post_attention_layernorm.weight._tp_sum_group = tp_group

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        qkv = self.qkv_proj(self.input_layernorm(x))                 # [T, local heads]
        T = qkv.shape[0]
        q, k, v = qkv.split([self.nq * self.hd, self.nkv * self.hd, self.nkv * self.hd], dim=-1)
        q = ops.rope_rotate_half(q.reshape(T, self.nq, self.hd), cos, sin)
        k = ops.rope_rotate_half(k.reshape(T, self.nkv, self.hd), cos, sin)
        o = ops.attention_varlen(q, k, v.reshape(T, self.nkv, self.hd), cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=True)
        x = x + self.o_proj(o.reshape(T, -1))
        return x + self.down_proj(ops.swiglu(self.gate_up_proj(self.post_attention_layernorm(x))))


class TPHead(nn.Module):
    def __init__(self, c: TextConfig, tp_group, sp: bool):
        super().__init__()
        self.group, self.sp = tp_group, sp
        tp = dist.get_world_size(tp_group) if tp_group is not None else 1
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.weight = nn.Parameter(torch.empty(c.vocab_size // tp, c.hidden_size))
        if sp and tp > 1:
            self.norm.weight._tp_sum_group = tp_group

    def forward(self, x, labels):
        h = self.norm(x)
        if self.sp:
            h = gather_sequence(h, self.group)
        else:
            from .tp import _CopyToTP
            if self.group is not None and dist.get_world_size(self.group) > 1:
                h = _CopyToTP.apply(h, self.group)
        logits = ops.linear(h, self.weight)
        return vocab_parallel_cross_entropy(logits, labels, self.group), (labels != -100).sum()


class McoreVLMStage(nn.Module):
    """The part of the VLM that lives on one (tp, pp) coordinate."""

    def __init__(self, cfg: Qwen25VLConfig, tp_group, pp_rank: int, pp_size: int, llm_layers: Sequence[int],
                 sequence_parallel: bool = True, vision_data_parallel: bool = False):
        super().__init__()
        self.cfg, self.tp_group, self.sp = cfg, tp_group, sequence_parallel
        self.vision_dp = vision_data_parallel and tp_group is not None
        self.first, self.last = pp_rank == 0, pp_rank == pp_size - 1
        self.layer_offset = sum(llm_layers[:pp_rank])
        t = cfg.text
        if self.first:
            self.visual = VisionTransformer(cfg.vision)
            if self.vision_dp:                  # ranks encode different images: sum the tower's gradients over them
                for p in self.visual.parameters():
                    p._tp_sum_group = tp_group
            self.embed_tokens = VocabParallelEmbedding(t.vocab_size, t.hidden_size, tp_group, sequence_parallel=False)
        self.layers = nn.ModuleList([TPDecoderLayer(t, tp_group, sequence_parallel) for _ in range(llm_layers[pp_rank])])
        if self.last:
            self.lm_head = TPHead(t, tp_group, sequence_parallel)

    def fsdp_units(self):
        units = []
        if self.first:
            units.append(("embed_tokens", self.embed_tokens))
            units.append(("visual.patch_embed", self.visual.patch_embed))
            units += [(f"visual.blocks.{i}", b) for i, b in enumerate(self.visual.blocks)]
            units.append(("visual.merger", self.visual.merger))
        units += [(f"layers.{self.layer_offset + i}", l) for i, l in enumerate(self.layers)]
        if self.last:
            units.append(("lm_head", self.lm_head))
        return units

    def forward(self, x_in, batch, run=None):
        run = run or (lambda m, *a, **k: m(*a, **k))
        t = self.cfg.text
        tp = dist.get_world_size(self.tp_group) if self.tp_group is not None else 1
        if self.first:
            ids = batch["input_ids"]
            x = run(self.embed_tokens, ids)
            pv = batch.get("pixel_values")
            if pv is not None and pv.numel() > 0:
                vis = self.visual
                share = None
                if self.vision_dp and tp > 1:
                    from .hetero import gather_image_rows, shard_images
                    grid = batch["image_grid_thw"]
                    share = shard_images(grid, tp, dist.get_rank(self.tp_group), vis.cfg.spatial_merge_size)
                if share is not None:
                    mine, rows, restore = share
                    cnt = grid.prod(-1)
                    off = torch.cumsum(cnt, 0) - cnt
                    pv = torch.cat([pv[int(off[i]):int(off[i] + cnt[i])] for i in mine])
                    plan = vis.plan(grid[mine], pv.device)
                else:
                    plan = batch.get("vision_plan") or vis.plan(batch["image_grid_thw"], pv.device)
                v = run(vis.patch_embed, pv.to(x.dtype)).index_select(0, plan["perm"])
                for i in range(len(vis.blocks)):
                    full = i in vis.cfg.fullatt_block_indexes
                    cu, mx = (plan["cu_full"], plan["max_full"]) if full else (plan["cu_win"], plan["max_win"])
                    v = run(vis.blocks[i], v, plan["cos"].to(x.dtype), plan["sin"].to(x.dtype), cu, mx)
                v = run(vis.merger, v).index_select(0, plan["reverse"])
                if share is not None:
                    v = gather_image_rows(v, rows, restore, self.tp_group)
                pos = batch.get("image_positions")
                if pos is None:
                    pos = (ids == self.cfg.image_token_id).nonzero(as_tuple=True)[0]
                x = x.index_copy(0, pos, v.to(x.dtype))
            if self.sp and tp > 1:
                x = split_sequence(x, self.tp_group)          # enter the sequence-parallel region
        else:
            x = x_in
        cos, sin = ops.ref.mrope_cos_sin(batch["position_ids"], t.head_dim, t.rope_theta, t.mrope_section)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        for layer in self.layers:
            x = run(layer, x, cos, sin, batch["cu_seqlens"], batch["max_seqlen"])
        if self.last:
            return run(self.lm_head, x, batch["labels"])
        return x


# ------------------------------------------------------------------------------------------ state sharding
def shard_full_state(full: Dict[str, torch.Tensor], cfg: Qwen25VLConfig, tp_rank: int, tp: int, pp_rank: int,
                     llm_layers: Sequence[int]) -> Dict[str, torch.Tensor]:
    """Local tensors of one (tp, pp) coordinate from a full internal-layout state dict (models/qwen2_5_vl.py names)."""
    t = cfg.text
    lo = sum(llm_layers[:pp_rank])
    hi = lo + llm_layers[pp_rank]
    pp = len(llm_layers)
    out: Dict[str, torch.Tensor] = {}

    def col(w):          # split output rows
        return w.chunk(tp, 0)[tp_rank].contiguous()

    def row(w):          # split input columns
        return w.chunk(tp, 1)[tp_rank].contiguous()

    for k, w in full.items():
        if k.startswith("visual.") or k == "embed_tokens.weight":
            if pp_rank == 0:
                out[k] = col(w) if k == "embed_tokens.weight" else w
        elif k.startswith("lm_head."):
            if pp_rank == pp - 1:
                out[k] = col(w) if k == "lm_head.weight" else w
        elif k.startswith("layers."):
            i = int(k.split(".")[1])
            if not lo <= i < hi:
                continue
            name = k.split(".", 2)[2]
            if name.startswith("qkv_proj."):
                qs, ks = t.num_attention_heads * t.head_dim, t.num_key_value_heads * t.head_dim
                q, kk, v = w.split([qs, ks, ks], 0)
                w2 = torch.cat([q.chunk(tp, 0)[tp_rank], kk.chunk(tp, 0)[tp_rank], v.chunk(tp, 0)[tp_rank]]).contiguous()
            elif name.startswith("gate_up_proj."):
                g, u = w.chunk(2, 0)
                w2 = torch.cat([g.chunk(tp, 0)[tp_rank], u.chunk(tp, 0)[tp_rank]]).contiguous()
            elif name in ("o_proj.weight", "down_proj.weight"):
                w2 = row(w)
            else:
                w2 = w
            out[k] = w2
    return out


# ------------------------------------------------------------------------------------------ driver
def build_mcore(cfg: Qwen25VLConfig, ps, device, opt, param_dtype, llm_layers=None, sequence_parallel=True,
                grad_accum_steps: int = 1, vision_data_parallel: bool = False):
    from .fsdp import FSDPEngine
    pp, tp = ps.size("pp"), ps.size("tp")
    layers = split_layers(cfg.text.num_layers, pp, llm_layers)
    with torch.device("meta"):
        stage = McoreVLMStage(cfg, ps.get_tp_group() if tp > 1 else None, ps.rank_in("pp"), pp, layers,
                              sequence_parallel and tp > 1, vision_data_parallel and tp > 1)
    dp = ps.size("dp")
    engine = FSDPEngine(stage.fsdp_units(), group=ps.group("dp") if dp > 1 else False, device=device,
                        param_dtype=param_dtype, opt=opt, grad_accum_steps=grad_accum_steps,
                        no_recompute=("lm_head",))
    return stage, engine, layers


def pretrain_mcore(kind: str, args, dev, rank: int, world: int):
    """Entry used by ``pretrain_vlm.py`` when --tensor-model-parallel-size / --pipeline-model-parallel-size > 1."""
    from ..api import stable_init_fn
    from ..data.collate import to_device
    from ..runtime.legacy_entry import datasets_provider
    from ..runtime.logging import format_training_log, print_rank0
    from ..runtime.lr_scheduler import LRSchedule
    from .fsdp import OptimConfig
    from .state import init_parallel_state
    import time
    if kind != "vlm":
        raise NotImplementedError("the TP/PP backend drives VLMs; DiTs use Ulysses/FSDP")
    tp, pp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size
    ps = init_parallel_state(world_size=world, device_type=dev.type, tensor_parallel_size=tp, pipeline_parallel_size=pp)
    cfg = Qwen25VLConfig.from_mm_json(args.mm.model.to_dict())
    td = args.mm.model.to_dict()["text_decoder"]
    accum = max(1, args.global_batch_size // (args.micro_batch_size * ps.size("dp")))
    opt = OptimConfig(lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                      weight_decay=args.weight_decay, clip_grad=0.0)
    stage, engine, layers = build_mcore(cfg, ps, dev, opt, torch.bfloat16 if (args.bf16 and dev.type == "cuda") else torch.float32,
                                        td.get("pipeline_num_layers"), bool(args.sequence_parallel), grad_accum_steps=accum,
                                        vision_data_parallel=bool(getattr(args, "hetero_parallel", False)))
    if getattr(args, "hetero_parallel", False) and tp > 1:
        from .hetero import HeteroPlan, ModulePlan
        print_rank0("> hetero parallel: " + HeteroPlan(world, {"vision": ModulePlan(pp=pp), "llm": ModulePlan(tp=tp, pp=pp)}).describe())
    engine.materialize(stable_init_fn(cfg.init_std, args.seed))
    pp_ranks = dist.get_process_group_ranks(ps.get_pp_group()) if pp > 1 else [rank]
    fwd_g = bwd_g = None
    if pp > 1:
        # every rank must take part in every new_group call
        all_pp = [None] * world
        dist.all_gather_object(all_pp, pp_ranks)
        for ranks in sorted({tuple(r) for r in all_pp}):
            a, b = dist.new_group(list(ranks)), dist.new_group(list(ranks))
            if rank in ranks:
                fwd_g, bwd_g = a, b
    tp_sz = tp if (args.sequence_parallel and tp > 1) else 1
    sched = PipelineSchedule(lambda c, x, mb: _stage_loss(stage, engine, x, mb, accum), ps.get_pp_group() if pp > 1 else None,
                             lambda mb: (mb["n_tokens"] // tp_sz, cfg.text.hidden_size), engine.param_dtype, dev,
                             fwd_group=fwd_g, bwd_group=bwd_g, after_backward=engine.end_micro_step)
    lr_s = LRSchedule(lr=args.lr, train_iters=args.train_iters, lr_decay_style=args.lr_decay_style,
                      lr_warmup_ratio=args.lr_warmup_fraction or 0.0, lr_min=args.min_lr or 0.0)
    data = datasets_provider(kind, args, type("M", (), {"config": cfg})(), ps)
    hist = []
    for it in range(args.train_iters):
        t0 = time.time()
        engine.set_lr(lr_s(it))
        mbs = [next(data) for _ in range(accum)]
        mbs = [to_device(m, dev) if dev.type == "cuda" else m for m in mbs]
        losses = sched.run(mbs)
        engine.finish_step()
        loss = torch.stack(losses).mean() if losses else torch.zeros((), device=dev)
        dist.all_reduce(loss)              # only last-stage ranks contribute; tp ranks of that stage each add it
        loss = loss / (tp * ps.size("dp"))
        hist.append(float(loss))
        print_rank0(format_training_log(it + 1, args.train_iters, (it + 1) * args.global_batch_size, time.time() - t0,
                                        lr_s(it), args.global_batch_size, {"loss": float(loss)}))
    return hist


def _stage_loss(stage, engine, x, mb, accum):
    out = stage(x, mb, run=engine.run)
    if isinstance(out, tuple):
        return out[0] / out[1].clamp(min=1)      # the engine averages over the accumulation steps
    return out
