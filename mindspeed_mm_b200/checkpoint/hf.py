"""HuggingFace-format weights: name maps, safetensors IO, load into / save from the sharding engine.

Internal parameter names are the modules' own (``layers.3.qkv_proj.weight``); HuggingFace names differ in
three ways that the operator list below undoes: prefixes (``model.language_model.`` / ``model.visual.`` in
current transformers, ``model.`` / ``visual.`` in older checkpoints), un-fused projections (q/k/v and
gate/up are separate tensors) and the Conv3d-shaped patch embedding.  Loading streams shard by shard and
writes straight into each rank's slice of the flat buffers (no full model is ever materialised on one
rank), the way the reference loads safetensors into sharded DTensors
(mindspeed_mm/fsdp/checkpoint/hf_utils.py:103-292); saving gathers unit by unit and writes size-capped
shards plus ``model.safetensors.index.json`` (hf_checkpointer.py:39-197).
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Sequence, Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .operators import (AddConst, ExpertStack, Merge, Operator, QKVMerge, Rename, RenamePrefix, Reshape, StateDict, Transpose,
                        apply_ops, revert_ops)

INDEX = "model.safetensors.index.json"


# ------------------------------------------------------------------------------------------ name maps
def qwen25vl_ops(cfg) -> List[Operator]:
    """HF Qwen2.5-VL -> internal names/layouts (``cfg``: models.qwen2_5_vl.Qwen25VLConfig)."""
    t, v = cfg.text, cfg.vision
    ffn, ffn_p = v.intermediate_size, (v.intermediate_size + 63) // 64 * 64

    def pad_rows(x, rows):      # [f, ...] -> [rows, ...] zero padded
        if x.shape[0] == rows:
            return x
        out = x.new_zeros((rows,) + tuple(x.shape[1:]))
        out[:x.shape[0]] = x
        return out

    class VitFFNPad(Operator):
        """Zero-pad the ViT FFN width (3420 -> 3456) after gate|up were merged; revert strips the pad."""

        def apply(self, sd):
            for k in list(sd.keys()):
                if k.startswith("visual.blocks.") and ".mlp_gate_up." in k:
                    g, u = torch.chunk(sd[k], 2, dim=0)
                    sd[k] = torch.cat([pad_rows(g, ffn_p), pad_rows(u, ffn_p)])
                elif k.startswith("visual.blocks.") and k.endswith("mlp_down.weight"):
                    w = sd[k]
                    if w.shape[1] != ffn_p:
                        out = w.new_zeros(w.shape[0], ffn_p)
                        out[:, :w.shape[1]] = w
                        sd[k] = out

        def revert(self, sd):
            for k in list(sd.keys()):
                if k.startswith("visual.blocks.") and ".mlp_gate_up." in k:
                    g, u = torch.chunk(sd[k], 2, dim=0)
                    sd[k] = torch.cat([g[:ffn], u[:ffn]])
                elif k.startswith("visual.blocks.") and k.endswith("mlp_down.weight"):
                    sd[k] = sd[k][:, :ffn].contiguous()

    ops: List[Operator] = [
        RenamePrefix("model.language_model.", "model."),       # current transformers layout -> classic
        RenamePrefix("model.visual.", "visual."),
        Rename("visual.patch_embed.proj.weight", "visual.patch_embed.proj.weight"),
        Reshape("visual.patch_embed.proj.weight", lambda x: (x.shape[0], -1),
                lambda x: (x.shape[0], v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)),
        Rename("visual.blocks.{i}.attn.qkv.weight", "visual.blocks.{i}.attn_qkv.weight"),
        Rename("visual.blocks.{i}.attn.qkv.bias", "visual.blocks.{i}.attn_qkv.bias"),
        Rename("visual.blocks.{i}.attn.proj.weight", "visual.blocks.{i}.attn_proj.weight"),
        Rename("visual.blocks.{i}.attn.proj.bias", "visual.blocks.{i}.attn_proj.bias"),
        Merge(["visual.blocks.{i}.mlp.gate_proj.weight", "visual.blocks.{i}.mlp.up_proj.weight"],
              "visual.blocks.{i}.mlp_gate_up.weight"),
        Merge(["visual.blocks.{i}.mlp.gate_proj.bias", "visual.blocks.{i}.mlp.up_proj.bias"],
              "visual.blocks.{i}.mlp_gate_up.bias"),
        Rename("visual.blocks.{i}.mlp.down_proj.weight", "visual.blocks.{i}.mlp_down.weight"),
        Rename("visual.blocks.{i}.mlp.down_proj.bias", "visual.blocks.{i}.mlp_down.bias"),
        VitFFNPad(),
        Rename("visual.merger.mlp.0.weight", "visual.merger.fc1.weight"),
        Rename("visual.merger.mlp.0.bias", "visual.merger.fc1.bias"),
        Rename("visual.merger.mlp.2.weight", "visual.merger.fc2.weight"),
        Rename("visual.merger.mlp.2.bias", "visual.merger.fc2.bias"),
        Rename("model.embed_tokens.weight", "embed_tokens.weight"),
        QKVMerge(["model.layers.{i}.self_attn.q_proj.weight", "model.layers.{i}.self_attn.k_proj.weight",
                  "model.layers.{i}.self_attn.v_proj.weight"], "layers.{i}.qkv_proj.weight",
                 t.num_attention_heads, t.num_key_value_heads, t.head_dim),
        QKVMerge(["model.layers.{i}.self_attn.q_proj.bias", "model.layers.{i}.self_attn.k_proj.bias",
                  "model.layers.{i}.self_attn.v_proj.bias"], "layers.{i}.qkv_proj.bias",
                 t.num_attention_heads, t.num_key_value_heads, t.head_dim),
        Rename("model.layers.{i}.self_attn.o_proj.weight", "layers.{i}.o_proj.weight"),
        Merge(["model.layers.{i}.mlp.gate_proj.weight", "model.layers.{i}.mlp.up_proj.weight"],
              "layers.{i}.gate_up_proj.weight"),
        Rename("model.layers.{i}.mlp.down_proj.weight", "layers.{i}.down_proj.weight"),
        Rename("model.layers.{i}.input_layernorm.weight", "layers.{i}.input_layernorm.weight"),
        Rename("model.layers.{i}.post_attention_layernorm.weight", "layers.{i}.post_attention_layernorm.weight"),
        Rename("model.norm.weight", "lm_head.norm.weight"),
        Rename("lm_head.weight", "lm_head.weight"),
    ]
    return ops


def qwen3vl_ops(cfg, experts_out_in: bool = False) -> List[Operator]:
    """HF Qwen3-VL / Qwen3-VL-MoE -> internal names/layouts (``cfg``: models.qwen3_vl.Qwen3VLConfig).

    Published MoE checkpoints store the fused experts as ``gate_up_proj [E, H, 2F]`` / ``down_proj [E, F, H]``, which is
    also the internal layout (reference: fsdp/models/qwen3vl/modeling_qwen3_vl_moe.py:125-126).  ``experts_out_in``
    reads / writes the ``[E, 2F, H]`` / ``[E, H, F]`` form that transformers >= 5 holds in memory instead."""
    t, v = cfg.text, cfg.vision
    ops: List[Operator] = [
        RenamePrefix("model.language_model.", "model."),
        RenamePrefix("model.visual.", "visual."),
        Reshape("visual.patch_embed.proj.weight", lambda x: (x.shape[0], -1),
                lambda x: (x.shape[0], v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)),
        Rename("visual.pos_embed.weight", "visual.patch_embed.pos_embed.weight"),
    ]
    for kind in ("weight", "bias"):
        ops += [
            Rename("visual.blocks.{i}.attn.qkv." + kind, "visual.blocks.{i}.attn_qkv." + kind),
            Rename("visual.blocks.{i}.attn.proj." + kind, "visual.blocks.{i}.attn_proj." + kind),
            Rename("visual.blocks.{i}.mlp.linear_fc1." + kind, "visual.blocks.{i}.mlp_fc1." + kind),
            Rename("visual.blocks.{i}.mlp.linear_fc2." + kind, "visual.blocks.{i}.mlp_fc2." + kind),
            Rename("visual.merger.linear_fc1." + kind, "visual.merger.fc1." + kind),
            Rename("visual.merger.linear_fc2." + kind, "visual.merger.fc2." + kind),
            Rename("visual.deepstack_merger_list.{i}.norm." + kind, "visual.deepstack_mergers.{i}.norm." + kind),
            Rename("visual.deepstack_merger_list.{i}.linear_fc1." + kind, "visual.deepstack_mergers.{i}.fc1." + kind),
            Rename("visual.deepstack_merger_list.{i}.linear_fc2." + kind, "visual.deepstack_mergers.{i}.fc2." + kind),
        ]
    ops += [
        Rename("model.embed_tokens.weight", "embed_tokens.weight"),
        QKVMerge(["model.layers.{i}.self_attn.q_proj.weight", "model.layers.{i}.self_attn.k_proj.weight",
                  "model.layers.{i}.self_attn.v_proj.weight"], "layers.{i}.qkv_proj.weight",
                 t.num_attention_heads, t.num_key_value_heads, t.head_dim),
        QKVMerge(["model.layers.{i}.self_attn.q_proj.bias", "model.layers.{i}.self_attn.k_proj.bias",
                  "model.layers.{i}.self_attn.v_proj.bias"], "layers.{i}.qkv_proj.bias",
                 t.num_attention_heads, t.num_key_value_heads, t.head_dim),
        Rename("model.layers.{i}.self_attn.o_proj.weight", "layers.{i}.o_proj.weight"),
        Rename("model.layers.{i}.self_attn.q_norm.weight", "layers.{i}.q_norm.weight"),
        Rename("model.layers.{i}.self_attn.k_norm.weight", "layers.{i}.k_norm.weight"),
        Merge(["model.layers.{i}.mlp.gate_proj.weight", "model.layers.{i}.mlp.up_proj.weight"],
              "layers.{i}.gate_up_proj.weight"),
        Rename("model.layers.{i}.mlp.down_proj.weight", "layers.{i}.down_proj.weight"),
        Rename("model.layers.{i}.mlp.gate.weight", "layers.{i}.mlp.gate.weight"),
        Rename("model.layers.{i}.mlp.experts.gate_up_proj", "layers.{i}.mlp.experts.gate_up_proj"),
        Rename("model.layers.{i}.mlp.experts.down_proj", "layers.{i}.mlp.experts.down_proj"),
        Rename("model.layers.{i}.input_layernorm.weight", "layers.{i}.input_layernorm.weight"),
        Rename("model.layers.{i}.post_attention_layernorm.weight", "layers.{i}.post_attention_layernorm.weight"),
        Rename("model.norm.weight", "lm_head.norm.weight"),
        Rename("lm_head.weight", "lm_head.weight"),
    ]
    if experts_out_in:
        ops += [Transpose("layers.{i}.mlp.experts.gate_up_proj"), Transpose("layers.{i}.mlp.experts.down_proj")]
    if t.tie_word_embeddings:
        ops.append(_UntieHead())
    return ops


def internvl_ops(cfg, experts_fused: bool = False) -> List[Operator]:
    """HF InternVL3 / InternVL3.5 (``model_type: internvl``) -> internal names/layouts (``cfg``:
    models.internvl.InternVLConfig): q | k | v of the tower and of the decoder are fused, gate | up fused, the patch
    convolution becomes a matmul over flattened patches.  Reference: checkpoint/vlm_model/converters/internvl.py."""
    t, v = cfg.text, cfg.vision
    V, B = "model.vision_tower.", "model.vision_tower.encoder.layer.{i}."
    L = "model.language_model.layers.{i}."
    ops: List[Operator] = [
        Reshape(V + "embeddings.patch_embeddings.projection.weight", lambda x: (x.shape[0], -1),
                lambda x: (x.shape[0], v.in_channels, v.patch_size, v.patch_size)),
        Rename(V + "embeddings.patch_embeddings.projection.weight", "visual.embed.proj.weight"),
        Rename(V + "embeddings.patch_embeddings.projection.bias", "visual.embed.proj.bias"),
        Rename(V + "embeddings.cls_token", "visual.embed.cls_token"),
        Rename(V + "embeddings.position_embeddings", "visual.embed.position_embeddings"),
        Rename(B + "lambda_1", "visual.blocks.{i}.lambda_1"),
        Rename(B + "lambda_2", "visual.blocks.{i}.lambda_2"),
        Rename(B + "attention.q_norm.weight", "visual.blocks.{i}.q_norm.weight"),
        Rename(B + "attention.k_norm.weight", "visual.blocks.{i}.k_norm.weight"),
    ]
    for kind in ("weight", "bias"):
        ops += [
            Merge([B + "attention.q_proj." + kind, B + "attention.k_proj." + kind, B + "attention.v_proj." + kind],
                  "visual.blocks.{i}.attn_qkv." + kind),
            Rename(B + "attention.projection_layer." + kind, "visual.blocks.{i}.attn_proj." + kind),
            Rename(B + "mlp.fc1." + kind, "visual.blocks.{i}.mlp_fc1." + kind),
            Rename(B + "mlp.fc2." + kind, "visual.blocks.{i}.mlp_fc2." + kind),
            Rename(B + "layernorm_before." + kind, "visual.blocks.{i}.norm1." + kind),
            Rename(B + "layernorm_after." + kind, "visual.blocks.{i}.norm2." + kind),
            Rename(V + "layernorm." + kind, "connector.norm." + kind),
            Rename("model.multi_modal_projector.layer_norm." + kind, "connector.projector.layer_norm." + kind),
            Rename("model.multi_modal_projector.linear_1." + kind, "connector.projector.linear_1." + kind),
            Rename("model.multi_modal_projector.linear_2." + kind, "connector.projector.linear_2." + kind),
            QKVMerge([L + "self_attn.q_proj." + kind, L + "self_attn.k_proj." + kind, L + "self_attn.v_proj." + kind],
                     "layers.{i}.qkv_proj." + kind, t.num_attention_heads, t.num_key_value_heads, t.head_dim),
        ]
    ops += [
        Rename("model.language_model.embed_tokens.weight", "embed_tokens.weight"),
        Rename(L + "self_attn.o_proj.weight", "layers.{i}.o_proj.weight"),
        Rename(L + "self_attn.q_norm.weight", "layers.{i}.q_norm.weight"),
        Rename(L + "self_attn.k_norm.weight", "layers.{i}.k_norm.weight"),
        Merge([L + "mlp.gate_proj.weight", L + "mlp.up_proj.weight"], "layers.{i}.gate_up_proj.weight"),
        Rename(L + "mlp.down_proj.weight", "layers.{i}.down_proj.weight"),
        Rename(L + "input_layernorm.weight", "layers.{i}.input_layernorm.weight"),
        Rename(L + "post_attention_layernorm.weight", "layers.{i}.post_attention_layernorm.weight"),
        Rename("model.language_model.norm.weight", "lm_head.norm.weight"),
        Rename("lm_head.weight", "lm_head.weight"),
    ]
    if t.num_experts:
        # published checkpoints list every expert (``experts.{e}.gate_proj.weight`` ...); transformers >= 5 holds them
        # fused as [E, 2F, H] / [E, H, F].  Internal layout: gate_up [E, H, 2F], down [E, F, H].
        E = L + "mlp.experts."
        ops += [Rename(L + "mlp.gate.weight", "layers.{i}.mlp.gate.weight")]
        if experts_fused:
            ops += [Rename(E + "gate_up_proj", "layers.{i}.mlp.experts.gate_up_proj"),
                    Rename(E + "down_proj", "layers.{i}.mlp.experts.down_proj"),
                    Transpose("layers.{i}.mlp.experts.gate_up_proj"), Transpose("layers.{i}.mlp.experts.down_proj")]
        else:
            ops += [Merge([E + "{e}.gate_proj.weight", E + "{e}.up_proj.weight"], E + "{e}.gate_up.weight"),
                    ExpertStack(E + "{e}.gate_up.weight", "layers.{i}.mlp.experts.gate_up_proj"),
                    ExpertStack(E + "{e}.down_proj.weight", "layers.{i}.mlp.experts.down_proj")]
    if t.tie_word_embeddings:
        ops.append(_UntieHead())
    return ops


def qwen35_ops(cfg, experts_out_in: bool = False) -> List[Operator]:
    """HF Qwen3.5 / Qwen3.5-MoE -> internal names/layouts (``cfg``: models.qwen3_5.Qwen35Config).  Beyond renames: the
    four input projections of a GDN layer are fused (q|k|v, z, b, a), its depthwise conv weight drops the singleton
    channel dim, q (with its per-head gate half) | k | v of a full-attention layer are fused, gate|up of the MLPs are
    fused, and the zero-centred RMSNorm weights of the text stack get their 1 back.  Reference:
    checkpoint/vlm_model/converters/qwen3_5.py."""
    t, v = cfg.text, cfg.vision
    L = "model.layers.{i}."
    ops: List[Operator] = [
        RenamePrefix("model.language_model.", "model."),
        RenamePrefix("model.visual.", "visual."),
        Reshape("visual.patch_embed.proj.weight", lambda x: (x.shape[0], -1),
                lambda x: (x.shape[0], v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)),
        Rename("visual.pos_embed.weight", "visual.patch_embed.pos_embed.weight"),
    ]
    for kind in ("weight", "bias"):
        ops += [
            Rename("visual.blocks.{i}.attn.qkv." + kind, "visual.blocks.{i}.attn_qkv." + kind),
            Rename("visual.blocks.{i}.attn.proj." + kind, "visual.blocks.{i}.attn_proj." + kind),
            Rename("visual.blocks.{i}.mlp.linear_fc1." + kind, "visual.blocks.{i}.mlp_fc1." + kind),
            Rename("visual.blocks.{i}.mlp.linear_fc2." + kind, "visual.blocks.{i}.mlp_fc2." + kind),
            Rename("visual.merger.linear_fc1." + kind, "visual.merger.fc1." + kind),
            Rename("visual.merger.linear_fc2." + kind, "visual.merger.fc2." + kind),
        ]
    ops += [
        Rename("model.embed_tokens.weight", "embed_tokens.weight"),
        # zero-centred norms first, under their HF names
        AddConst(L + "input_layernorm.weight"), AddConst(L + "post_attention_layernorm.weight"),
        AddConst(L + "self_attn.q_norm.weight"), AddConst(L + "self_attn.k_norm.weight"), AddConst("model.norm.weight"),
        # GDN
        Merge([L + "linear_attn.in_proj_qkv.weight", L + "linear_attn.in_proj_z.weight", L + "linear_attn.in_proj_b.weight",
               L + "linear_attn.in_proj_a.weight"], "layers.{i}.linear_attn.in_proj.weight",
              sizes=[2 * t.linear_num_key_heads * t.linear_key_head_dim + t.linear_num_value_heads * t.linear_value_head_dim,
                     t.linear_num_value_heads * t.linear_value_head_dim, t.linear_num_value_heads, t.linear_num_value_heads]),
        Reshape(L + "linear_attn.conv1d.weight", lambda x: (x.shape[0], x.shape[-1]), lambda x: (x.shape[0], 1, x.shape[-1])),
        Rename(L + "linear_attn.conv1d.weight", "layers.{i}.linear_attn.conv_weight"),
        Rename(L + "linear_attn.dt_bias", "layers.{i}.linear_attn.dt_bias"),
        Rename(L + "linear_attn.A_log", "layers.{i}.linear_attn.A_log"),
        Rename(L + "linear_attn.norm.weight", "layers.{i}.linear_attn.norm_weight"),
        Rename(L + "linear_attn.out_proj.weight", "layers.{i}.linear_attn.out_proj.weight"),
        # gated attention: q_proj holds query|gate per head, i.e. 2 x heads "heads" for the split sizes
        QKVMerge([L + "self_attn.q_proj.weight", L + "self_attn.k_proj.weight", L + "self_attn.v_proj.weight"],
                 "layers.{i}.self_attn.qkv_proj.weight", t.num_attention_heads * (2 if t.attn_output_gate else 1),
                 t.num_key_value_heads, t.head_dim),
        Rename(L + "self_attn.o_proj.weight", "layers.{i}.self_attn.o_proj.weight"),
        Rename(L + "self_attn.q_norm.weight", "layers.{i}.self_attn.q_norm.weight"),
        Rename(L + "self_attn.k_norm.weight", "layers.{i}.self_attn.k_norm.weight"),
        # FFNs
        Merge([L + "mlp.gate_proj.weight", L + "mlp.up_proj.weight"], "layers.{i}.gate_up_proj.weight"),
        Rename(L + "mlp.down_proj.weight", "layers.{i}.down_proj.weight"),
        Rename(L + "mlp.gate.weight", "layers.{i}.mlp.routed.gate.weight"),
        Rename(L + "mlp.experts.gate_up_proj", "layers.{i}.mlp.routed.experts.gate_up_proj"),
        Rename(L + "mlp.experts.down_proj", "layers.{i}.mlp.routed.experts.down_proj"),
        Merge([L + "mlp.shared_expert.gate_proj.weight", L + "mlp.shared_expert.up_proj.weight"],
              "layers.{i}.mlp.shared_gate_up.weight"),
        Rename(L + "mlp.shared_expert.down_proj.weight", "layers.{i}.mlp.shared_down.weight"),
        Rename(L + "mlp.shared_expert_gate.weight", "layers.{i}.mlp.shared_expert_gate.weight"),
        Rename(L + "input_layernorm.weight", "layers.{i}.input_layernorm.weight"),
        Rename(L + "post_attention_layernorm.weight", "layers.{i}.post_attention_layernorm.weight"),
        Rename("model.norm.weight", "lm_head.norm.weight"),
        Rename("lm_head.weight", "lm_head.weight"),
    ]
    if experts_out_in:
        ops += [Transpose("layers.{i}.mlp.routed.experts.gate_up_proj"), Transpose("layers.{i}.mlp.routed.experts.down_proj")]
    if t.tie_word_embeddings:
        ops.append(_UntieHead())
    return ops


def hunyuanvideo_ops(cfg) -> List[Operator]:
    """Published HunyuanVideo transformer checkpoint (``double_blocks.N.img_mod.linear``, ``txt_in.individual_token_refiner``,
    ``final_layer`` ...) -> internal names (``cfg``: models.mmdit.MMDiTConfig).  The patch embedding is a Conv3d whose
    kernel equals its stride, i.e. a Linear over flattened patches; everything else is a rename.  Reference:
    checkpoint/sora_model/hunyuanvideo_converter.py:31-60 (its target names differ, the source names are the same)."""
    p = cfg.patch_size
    ops: List[Operator] = [
        Reshape("img_in.proj.weight", lambda x: (x.shape[0], -1), lambda x: (x.shape[0], cfg.in_channels, p[0], p[1], p[2])),
    ]
    wb = ("weight", "bias")
    pairs = [("img_in.proj", "embed.img_in"), ("time_in.mlp.0", "embed.time_in_0"), ("time_in.mlp.2", "embed.time_in_2"),
             ("vector_in.in_layer", "embed.vector_in_0"), ("vector_in.out_layer", "embed.vector_in_2"),
             ("guidance_in.mlp.0", "embed.guidance_in_0"), ("guidance_in.mlp.2", "embed.guidance_in_2"),
             ("txt_in.input_embedder", "embed.txt_in.input_embedder"),
             ("txt_in.t_embedder.mlp.0", "embed.txt_in.t_0"), ("txt_in.t_embedder.mlp.2", "embed.txt_in.t_2"),
             ("txt_in.c_embedder.linear_1", "embed.txt_in.c_1"), ("txt_in.c_embedder.linear_2", "embed.txt_in.c_2"),
             ("final_layer.linear", "final.linear"), ("final_layer.adaLN_modulation.1", "final.mod.lin")]
    R, B = "txt_in.individual_token_refiner.blocks.{i}.", "embed.txt_in.blocks.{i}."
    pairs += [(R + "norm1", B + "norm1"), (R + "norm2", B + "norm2"), (R + "self_attn_qkv", B + "qkv"),
              (R + "self_attn_proj", B + "proj"), (R + "mlp.fc1", B + "mlp_0"), (R + "mlp.fc2", B + "mlp_2"),
              (R + "adaLN_modulation.1", B + "mod")]
    for st in ("img", "txt"):
        D, I = "double_blocks.{i}." + st + "_", "double_blocks.{i}." + st + "."
        pairs += [(D + "mod.linear", I + "mod.lin"), (D + "attn_qkv", I + "qkv"), (D + "attn_proj", I + "proj"),
                  (D + "mlp.fc1", I + "mlp_0"), (D + "mlp.fc2", I + "mlp_2")]
        ops += [Rename(D + "attn_q_norm.weight", I + "q_norm.weight"), Rename(D + "attn_k_norm.weight", I + "k_norm.weight")]
    pairs += [("single_blocks.{i}.modulation.linear", "single_blocks.{i}.mod.lin")]      # linear1 / linear2 / q_norm / k_norm keep their names
    for a, b in pairs:
        ops += [Rename(f"{a}.{k}", f"{b}.{k}") for k in wb]
    return ops


class _UntieHead(Operator):
    """A tied checkpoint has no ``lm_head.weight``: the internal head gets a copy of the embedding; the way back
    drops it again."""

    def apply(self, sd):
        if "lm_head.weight" not in sd and "embed_tokens.weight" in sd:
            sd["lm_head.weight"] = sd["embed_tokens.weight"].clone()

    def revert(self, sd):
        sd.pop("lm_head.weight", None)


class _ModernPrefix(Operator):
    """On the way back to HF, emit the current transformers prefixes."""

    def apply(self, sd):
        pass

    def revert(self, sd):
        for k in list(sd.keys()):
            if k.startswith("model."):
                sd["model.language_model." + k[len("model."):]] = sd.pop(k)
            elif k.startswith("visual."):
                sd["model." + k] = sd.pop(k)


def to_internal(hf_sd: StateDict, ops: List[Operator]) -> StateDict:
    return apply_ops(dict(hf_sd), ops)


class UnderPrefix(Operator):
    """Internal name = ``prefix`` + the checkpoint's own name, nothing else changes (models wrapped as they are, e.g.
    ``plugins/hf_adapter.py``).  Marks the operator list as exact: no prefix modernisation on the way back."""

    exact_names = True

    def __init__(self, prefix: str):
        self.prefix = prefix

    def apply(self, sd):
        for k in list(sd.keys()):
            sd[self.prefix + k] = sd.pop(k)

    def revert(self, sd):
        for k in list(sd.keys()):
            if k.startswith(self.prefix):
                sd[k[len(self.prefix):]] = sd.pop(k)


class MatchBySuffix(Operator):
    """Checkpoint names -> the names of a model built by the current transformers version, for files written with an
    older layout of the same architecture (``model.layers...`` / ``visual...`` or ``language_model.model.layers...`` on
    disk, ``model.language_model.layers...`` / ``model.visual...`` in memory).  A name the model does not have is replaced
    by the one model name that ends with the longest possible tail of it; when several do, the components that were cut off
    (other than the generic ``model``) must all appear in the candidate.  Names that still match nothing, or more than one,
    are left alone.  The way back writes the model's own names, which every transformers version that knows them reads."""

    exact_names = True

    def __init__(self, model_names: Sequence[str]):
        self.names = list(model_names)

    def apply(self, sd):
        have = set(self.names)
        free = [n for n in self.names if n not in sd]
        for k in list(sd.keys()):
            if k in have:
                continue
            parts = k.split(".")
            for drop in range(0, len(parts) - 1):
                tail = "." + ".".join(parts[drop:])
                hits = [n for n in free if n.endswith(tail)]
                if len(hits) > 1:
                    hint = [c for c in parts[:drop] if c != "model"]
                    hits = [n for n in hits if all(c in n.split(".") for c in hint)]
                if len(hits) == 1:
                    sd[hits[0]] = sd.pop(k)
                    free.remove(hits[0])
                    break
                if hits:            # still ambiguous at this length: a shorter tail can only be more so
                    break

    def revert(self, sd):
        pass


def to_hf(internal_sd: StateDict, ops: List[Operator], modern_prefix: bool = True) -> StateDict:
    modern_prefix = modern_prefix and not any(getattr(o, "exact_names", False) for o in ops)
    ops = [o for o in ops if not isinstance(o, RenamePrefix)]
    sd = revert_ops(dict(internal_sd), ops)
    if modern_prefix:
        _ModernPrefix().revert(sd)
    return sd


# ------------------------------------------------------------------------------------------ safetensors IO
def iter_safetensors(path: str) -> Iterable[Tuple[str, torch.Tensor]]:
    """Yield (name, tensor) from a file, a sharded directory (index json) or a directory of *.safetensors."""
    from safetensors import safe_open
    files: List[str]
    if os.path.isfile(path):
        files = [path]
    else:
        idx = os.path.join(path, INDEX)
        if os.path.exists(idx):
            with open(idx) as f:
                files = sorted({os.path.join(path, v) for v in json.load(f)["weight_map"].values()})
        else:
            files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
    for fp in files:
        with safe_open(fp, framework="pt", device="cpu") as f:
            for k in f.keys():
                yield k, f.get_tensor(k)


def load_state_dict(path: str) -> StateDict:
    return dict(iter_safetensors(path))


def save_sharded(sd: StateDict, out_dir: str, max_shard_bytes: int = 5 << 30, metadata: Optional[dict] = None) -> None:
    from safetensors.torch import save_file
    os.makedirs(out_dir, exist_ok=True)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k in sorted(sd):
        t = sd[k].contiguous()
        nb = t.numel() * t.element_size()
        if size + nb > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][k] = t
        size += nb
    weight_map, total = {}, 0
    n = len(shards)
    for i, sh in enumerate(shards):
        name = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
        save_file(sh, os.path.join(out_dir, name), metadata={"format": "pt"})
        for k, t in sh.items():
            weight_map[k] = name
            total += t.numel() * t.element_size()
    if n > 1:
        with open(os.path.join(out_dir, INDEX), "w") as f:
            json.dump({"metadata": {"total_size": total, **(metadata or {})}, "weight_map": weight_map}, f, indent=2)


def is_hf_checkpoint(path: str) -> bool:
    if not path or not os.path.isdir(path):
        return False
    return any(f.endswith(".safetensors") for f in os.listdir(path))


# ------------------------------------------------------------------------------------------ engine bridges
def load_hf_into_engine(engine, path: str, ops: List[Operator], strict: bool = True) -> List[str]:
    """Fill the engine's shards from an HF checkpoint.  Returns missing internal names."""
    sd = to_internal(load_state_dict(path), ops)

    def getter(name, shape):
        t = sd.get(name)
        if t is None and ".base." in name:          # a LoRA-wrapped linear keeps the checkpoint's weight as its frozen base
            t = sd.get(name.replace(".base.", "."))
        if t is None:
            return None
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(t.shape)} vs model {tuple(shape)}")
        return t.to(engine.device)

    missing = engine.load_full_params(getter)
    if strict and missing:
        raise KeyError(f"missing in checkpoint: {missing[:8]}{'...' if len(missing) > 8 else ''}")
    return missing


def save_engine_as_hf(engine, out_dir: str, ops: List[Operator], dtype: Optional[torch.dtype] = None,
                      assets_from: Optional[str] = None, rank: int = 0) -> None:
    """Gather unit by unit (all ranks participate); rank 0 writes the HF-named safetensors shards and copies
    tokenizer / config assets from ``assets_from``."""
    sd: StateDict = {}
    for name, t in engine.named_full_params():
        if rank == 0:
            sd[name] = (t.to(dtype) if dtype else t).detach().cpu().clone()
    if rank == 0:
        save_sharded(to_hf(sd, ops), out_dir)
        if assets_from and os.path.isdir(assets_from):
            for f in os.listdir(assets_from):
                if f.endswith((".json", ".txt", ".model", ".jinja")) and f != INDEX:
                    shutil.copy(os.path.join(assets_from, f), os.path.join(out_dir, f))
