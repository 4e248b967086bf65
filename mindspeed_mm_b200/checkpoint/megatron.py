"""Megatron-format ("MM") checkpoints and the HF <-> MM converters for Qwen2/2.5-VL.

Directory layout written and read here (what the reference's mcore path loads,
checkpoint/vlm_model/hf_to_mm.py:60-62,168-195):

    <dir>/latest_checkpointed_iteration.txt                    "release" or an iteration number
    <dir>/<release|iter_XXXXXXX>/mp_rank_{tp:02d}[_{pp:03d}][_{ep:03d}]/model_optim_rng.pt
        {"model" | "model0","model1",... (virtual pipeline chunks): state_dict, "checkpoint_version": 3.0}

Conversion = name/layout operators (HF names -> Megatron names, q|k|v interleaved per KV group, gate|up
concatenated, ViT qkv interleaved per head) -> tensor-parallel split (column / row / GLU rules) ->
pipeline partition with per-stage layer renumbering (``pipeline_num_layers`` lists for the ViT and the LLM;
a stage with 0 layers of a module simply holds none of it) -> one file per (tp, pp) rank.  ``mm_to_hf`` is the
exact inverse and ``resplit`` is mm_to_hf followed by hf_to_mm in memory.  Name map:
checkpoint/vlm_model/converters/qwen2vl.py:21-105 and qwen2_5vl.py:21-49; split rules: qwen2vl.py:108-149.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .operators import (Merge, Operator, QKVMerge, Rename, RenamePrefix, StateDict, apply_ops, concat_to_interleaved,
                        interleaved_to_concat, merge_glu, revert_ops, split_col, split_glu, split_row)

CHECKPOINT_VERSION = 3.0
TRACKER = "latest_checkpointed_iteration.txt"


class HeadInterleave(Operator):
    """ViT fused qkv: HF stores [q_all | k_all | v_all]; Megatron wants [q_h0,k_h0,v_h0, q_h1, ...]."""

    def __init__(self, pattern: str, num_heads: int):
        self.rx, self.nh = re.compile(pattern), num_heads

    def apply(self, sd):
        for k in list(sd.keys()):
            if self.rx.fullmatch(k):
                third = sd[k].shape[0] // 3
                sd[k] = concat_to_interleaved(sd[k], self.nh, [third] * 3)

    def revert(self, sd):
        for k in list(sd.keys()):
            if self.rx.fullmatch(k):
                hd = sd[k].shape[0] // 3 // self.nh
                sd[k] = interleaved_to_concat(sd[k], self.nh, [hd] * 3)


def qwen25vl_mm_ops(num_heads: int, num_kv_heads: int, head_dim: int, vit_heads: int, glu_vit: bool = True) -> List[Operator]:
    v, t = "image_encoder.encoder.blocks.layers.{i}.", "text_decoder.decoder.layers.{i}."
    ops: List[Operator] = [RenamePrefix("model.language_model.", "model."), RenamePrefix("model.visual.", "visual.")]
    if glu_vit:   # Qwen2.5-VL: gated ViT MLP
        ops += [Merge(["visual.blocks.{i}.mlp.gate_proj.weight", "visual.blocks.{i}.mlp.up_proj.weight"], v + "mlp.linear_fc1.weight"),
                Merge(["visual.blocks.{i}.mlp.gate_proj.bias", "visual.blocks.{i}.mlp.up_proj.bias"], v + "mlp.linear_fc1.bias"),
                Rename("visual.blocks.{i}.mlp.down_proj.weight", v + "mlp.linear_fc2.weight"),
                Rename("visual.blocks.{i}.mlp.down_proj.bias", v + "mlp.linear_fc2.bias")]
    else:         # Qwen2-VL: fc1 / fc2
        ops += [Rename("visual.blocks.{i}.mlp.fc1." + s, v + "mlp.linear_fc1." + s) for s in ("weight", "bias")]
        ops += [Rename("visual.blocks.{i}.mlp.fc2." + s, v + "mlp.linear_fc2." + s) for s in ("weight", "bias")]
    for s in ("weight", "bias"):
        ops += [Rename("visual.blocks.{i}.attn.proj." + s, v + "self_attention.linear_proj." + s),
                Rename("visual.blocks.{i}.attn.qkv." + s, v + "self_attention.linear_qkv." + s),
                Rename("visual.merger.mlp.0." + s, "image_encoder.projector.encoder.linear_fc1." + s),
                Rename("visual.merger.mlp.2." + s, "image_encoder.projector.encoder.linear_fc2." + s),
                Rename("visual.blocks.{i}.norm1." + s, v + "input_layernorm." + s),
                Rename("visual.blocks.{i}.norm2." + s, v + "pre_mlp_layernorm." + s),
                Rename("visual.merger.ln_q." + s, "image_encoder.projector.layernorm." + s)]
    ops += [HeadInterleave(r"image_encoder\.encoder\.blocks\.layers\.\d+\.self_attention\.linear_qkv\.(weight|bias)", vit_heads),
            Rename("visual.patch_embed.proj.weight", "image_encoder.encoder.patch_embed.proj.weight"),
            Rename("model.embed_tokens.weight", "text_decoder.embedding.word_embeddings.weight"),
            Rename("model.layers.{i}.input_layernorm.weight", t + "input_layernorm.weight"),
            Rename("model.layers.{i}.post_attention_layernorm.weight", t + "pre_mlp_layernorm.weight"),
            Rename("model.layers.{i}.mlp.down_proj.weight", t + "mlp.linear_fc2.weight"),
            Rename("model.layers.{i}.self_attn.o_proj.weight", t + "self_attention.linear_proj.weight"),
            Merge(["model.layers.{i}.mlp.gate_proj.weight", "model.layers.{i}.mlp.up_proj.weight"], t + "mlp.linear_fc1.weight"),
            QKVMerge(["model.layers.{i}.self_attn.%s_proj.weight" % x for x in "qkv"], t + "self_attention.linear_qkv.weight",
                     num_heads, num_kv_heads, head_dim, interleave_groups=True),
            QKVMerge(["model.layers.{i}.self_attn.%s_proj.bias" % x for x in "qkv"], t + "self_attention.linear_qkv.bias",
                     num_heads, num_kv_heads, head_dim, interleave_groups=True),
            Rename("lm_head.weight", "text_decoder.output_layer.weight"),
            Rename("model.norm.weight", "text_decoder.decoder.final_layernorm.weight")]
    return ops


# (pattern, rule): "row" = split dim 0 (column-parallel / vocab-parallel), "col" = split dim 1 (row-parallel)
QWEN2VL_TP_RULES: List[Tuple[str, str]] = [
    (r"text_decoder\.output_layer\.weight", "row"),
    (r"text_decoder\.embedding\.word_embeddings\.weight", "row"),
    (r"text_decoder\.decoder\.layers\.\d+\.mlp\.linear_fc2\.weight", "col"),
    (r"text_decoder\.decoder\.layers\.\d+\.self_attention\.linear_proj\.weight", "col"),
    (r"text_decoder\.decoder\.layers\.\d+\.mlp\.linear_fc1\.weight", "glu"),
    (r"text_decoder\.decoder\.layers\.\d+\.self_attention\.linear_qkv\.(weight|bias)", "row"),
    (r"image_encoder\.encoder\.blocks\.layers\.\d+\.self_attention\.linear_proj\.weight", "col"),
    (r"image_encoder\.encoder\.blocks\.layers\.\d+\.self_attention\.linear_qkv\.(weight|bias)", "row"),
    (r"image_encoder\.encoder\.blocks\.layers\.\d+\.mlp\.linear_fc1\.(weight|bias)", "row"),
    (r"image_encoder\.encoder\.blocks\.layers\.\d+\.mlp\.linear_fc2\.weight", "col"),
    (r"image_encoder\.projector\.encoder\.linear_fc1\.(weight|bias)", "row"),
    (r"image_encoder\.projector\.encoder\.linear_fc2\.weight", "col"),
]


def split_by_tp(sd: StateDict, tp: int, rules=QWEN2VL_TP_RULES, glu_vit: bool = True) -> List[StateDict]:
    if tp == 1:
        return [dict(sd)]
    outs: List[StateDict] = [dict() for _ in range(tp)]
    comp = [(re.compile(p), r) for p, r in rules]
    for k, t in sd.items():
        rule = next((r for rx, r in comp if rx.fullmatch(k)), None)
        if rule == "glu" and "image_encoder" in k and not glu_vit:
            rule = "row"
        parts = {"row": lambda: split_col(t, tp), "col": lambda: split_row(t, tp), "glu": lambda: split_glu(t, tp),
                 None: lambda: [t] * tp}[rule]()
        for r in range(tp):
            outs[r][k] = parts[r]
    return outs


def merge_by_tp(sds: Sequence[StateDict], rules=QWEN2VL_TP_RULES, glu_vit: bool = True) -> StateDict:
    if len(sds) == 1:
        return dict(sds[0])
    comp = [(re.compile(p), r) for p, r in rules]
    out: StateDict = {}
    for k in sds[0]:
        rule = next((r for rx, r in comp if rx.fullmatch(k)), None)
        if rule == "glu" and "image_encoder" in k and not glu_vit:
            rule = "row"
        parts = [sd[k] for sd in sds]
        if rule == "row":
            out[k] = torch.cat(parts, 0)
        elif rule == "col":
            out[k] = torch.cat(parts, 1) if parts[0].dim() > 1 else parts[0]
        elif rule == "glu":
            out[k] = merge_glu(parts)
        else:
            out[k] = parts[0]
    return out


@dataclass
class StageSchema:
    firsts: Tuple[str, ...]
    lasts: Tuple[str, ...]
    middle: str


TEXT = StageSchema(("text_decoder.embedding.",), ("text_decoder.decoder.final_layernorm.", "text_decoder.output_layer."),
                   "text_decoder.decoder.layers.")
VISION = StageSchema(("image_encoder.encoder.patch_embed.",), ("image_encoder.projector.",),
                     "image_encoder.encoder.blocks.layers.")


def partition_by_pp(sd: StateDict, layer_lists: Sequence[Sequence[int]], schemas: Sequence[StageSchema]) -> List[StateDict]:
    """``layer_lists[m][p]`` = layers of module m on pipeline stage p.  A module's first-stage tensors go to
    the first stage that holds any of its layers, its last-stage tensors to the last such stage; layer
    indices are renumbered from 0 on every stage."""
    pp = len(layer_lists[0])
    outs: List[StateDict] = [dict() for _ in range(pp)]
    for layers, sc in zip(layer_lists, schemas):
        holders = [p for p in range(pp) if layers[p] > 0]
        first, last = holders[0], holders[-1]
        starts = [sum(layers[:p]) for p in range(pp)]
        rx = re.compile(re.escape(sc.middle) + r"(\d+)\.(.*)")
        for k, t in sd.items():
            if any(k.startswith(f) for f in sc.firsts):
                outs[first][k] = t
            elif any(k.startswith(f) for f in sc.lasts):
                outs[last][k] = t
            else:
                m = rx.fullmatch(k)
                if m:
                    li = int(m.group(1))
                    for p in range(pp):
                        if starts[p] <= li < starts[p] + layers[p]:
                            outs[p][f"{sc.middle}{li - starts[p]}.{m.group(2)}"] = t
    return outs


def merge_pp(stage_sds: Sequence[StateDict], layer_lists: Sequence[Sequence[int]], schemas: Sequence[StageSchema]) -> StateDict:
    out: StateDict = {}
    for p, sd in enumerate(stage_sds):
        for k, t in sd.items():
            placed = False
            for layers, sc in zip(layer_lists, schemas):
                m = re.fullmatch(re.escape(sc.middle) + r"(\d+)\.(.*)", k)
                if m:
                    out[f"{sc.middle}{int(m.group(1)) + sum(layers[:p])}.{m.group(2)}"] = t
                    placed = True
                    break
            if not placed:
                out[k] = t
    return out


def rank_dir(root: str, tp: int, pp: Optional[int] = None, ep: Optional[int] = None) -> str:
    name = f"mp_rank_{tp:02d}"
    if pp is not None:
        name += f"_{pp:03d}"
    if ep is not None:
        name += f"_{ep:03d}"
    return os.path.join(root, name)


def save_mm(stage_tp_sds: List[List[StateDict]], out_dir: str, iteration: Optional[int] = None) -> None:
    """``stage_tp_sds[pp][tp]`` -> files.  ``iteration=None`` writes a ``release`` checkpoint."""
    tag = "release" if iteration is None else f"iter_{iteration:07d}"
    pp_size = len(stage_tp_sds)
    for pp, per_tp in enumerate(stage_tp_sds):
        for tp, sd in enumerate(per_tp):
            d = rank_dir(os.path.join(out_dir, tag), tp, pp if pp_size > 1 else None)
            os.makedirs(d, exist_ok=True)
            torch.save({"model": sd, "checkpoint_version": CHECKPOINT_VERSION}, os.path.join(d, "model_optim_rng.pt"))
    with open(os.path.join(out_dir, TRACKER), "w") as f:
        f.write("release" if iteration is None else str(iteration))


def load_mm(in_dir: str) -> List[List[StateDict]]:
    tag = open(os.path.join(in_dir, TRACKER)).read().strip()
    root = os.path.join(in_dir, tag if tag == "release" else f"iter_{int(tag):07d}")
    found: Dict[Tuple[int, int], StateDict] = {}
    for name in os.listdir(root):
        m = re.fullmatch(r"mp_rank_(\d+)(?:_(\d+))?(?:_(\d+))?", name)
        if m:
            ck = torch.load(os.path.join(root, name, "model_optim_rng.pt"), map_location="cpu", weights_only=False)
            found[(int(m.group(2) or 0), int(m.group(1)))] = ck["model"]
    pp, tp = max(k[0] for k in found) + 1, max(k[1] for k in found) + 1
    return [[found[(p, t)] for t in range(tp)] for p in range(pp)]


def hf_to_mm(hf_sd: StateDict, ops: List[Operator], tp: int, vit_layers: Sequence[int], llm_layers: Sequence[int],
             glu_vit: bool = True) -> List[List[StateDict]]:
    sd = apply_ops(dict(hf_sd), ops)
    per_tp = split_by_tp(sd, tp, glu_vit=glu_vit)
    stages_per_tp = [partition_by_pp(s, [vit_layers, llm_layers], [VISION, TEXT]) for s in per_tp]
    pp = len(llm_layers)
    return [[stages_per_tp[t][p] for t in range(tp)] for p in range(pp)]


def mm_to_hf(stage_tp_sds: List[List[StateDict]], ops: List[Operator], vit_layers: Sequence[int],
             llm_layers: Sequence[int], glu_vit: bool = True, modern_prefix: bool = True) -> StateDict:
    tp = len(stage_tp_sds[0])
    per_tp = [merge_pp([stage_tp_sds[p][t] for p in range(len(stage_tp_sds))], [vit_layers, llm_layers], [VISION, TEXT])
              for t in range(tp)]
    sd = merge_by_tp(per_tp, glu_vit=glu_vit)
    sd = revert_ops(sd, [o for o in ops if not isinstance(o, RenamePrefix)])
    if modern_prefix:
        for k in list(sd.keys()):
            if k.startswith("model."):
                sd["model.language_model." + k[6:]] = sd.pop(k)
            elif k.startswith("visual."):
                sd["model." + k] = sd.pop(k)
    return sd
