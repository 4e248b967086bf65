"""Wan2.1 weight names: diffusers ``WanTransformer3DModel`` <-> Megatron-side ("MM") names <-> this package.

MM names are the reference's (checkpoint/sora_model/wan_converter.py:29-76): ``blocks.N.self_attn.proj_q`` ...,
``time_embedding.0/2``, ``time_projection.1``, ``text_embedding.linear_1/2``, ``head.head``, ``head.modulation``.
Internally q|k|v of self-attention and k|v of cross-attention are fused into one GEMM each, and the
embeddings live in one unit; ``mm_to_internal`` / ``internal_to_mm`` do that last hop.
"""
from __future__ import annotations

from typing import Dict

import torch

from .operators import Merge, Rename, StateDict, apply_ops, revert_ops

_EXACT = {
    "condition_embedder.text_embedder.linear_1.": "text_embedding.linear_1.",
    "condition_embedder.text_embedder.linear_2.": "text_embedding.linear_2.",
    "condition_embedder.time_embedder.linear_1.": "time_embedding.0.",
    "condition_embedder.time_embedder.linear_2.": "time_embedding.2.",
    "condition_embedder.time_proj.": "time_projection.1.",
    "condition_embedder.image_embedder.ff.net.0.proj.": "img_emb.proj.1.",
    "condition_embedder.image_embedder.ff.net.2.": "img_emb.proj.3.",
    "condition_embedder.image_embedder.norm1.": "img_emb.proj.0.",
    "condition_embedder.image_embedder.norm2.": "img_emb.proj.4.",
    "condition_embedder.image_embedder.pos_embed": "img_emb.emb_pos",
    "proj_out.": "head.head.",
}
_SUBSTR = [
    ("attn1.norm_q", "self_attn.q_norm"), ("attn1.norm_k", "self_attn.k_norm"),
    ("attn2.norm_q", "cross_attn.q_norm"), ("attn2.norm_k", "cross_attn.k_norm"),
    ("attn1.to_q.", "self_attn.proj_q."), ("attn1.to_k.", "self_attn.proj_k."), ("attn1.to_v.", "self_attn.proj_v."),
    ("attn1.to_out.0.", "self_attn.proj_out."),
    ("attn2.to_q.", "cross_attn.proj_q."), ("attn2.to_k.", "cross_attn.proj_k."), ("attn2.to_v.", "cross_attn.proj_v."),
    ("attn2.add_k_proj", "cross_attn.k_img"), ("attn2.add_v_proj", "cross_attn.v_img"),
    ("attn2.norm_added_k", "cross_attn.k_norm_img"), ("attn2.to_out.0.", "cross_attn.proj_out."),
    (".ffn.net.0.proj.", ".ffn.0."), (".ffn.net.2.", ".ffn.2."), (".norm2.", ".norm3."),
]


def diffusers_to_mm(sd: StateDict) -> StateDict:
    out = {}
    for k, v in sd.items():
        if k == "scale_shift_table":
            out["head.modulation"] = v
            continue
        nk = k
        for a, b in _EXACT.items():
            if nk.startswith(a):
                nk = b + nk[len(a):]
                break
        else:
            for a, b in _SUBSTR:
                nk = nk.replace(a, b)
            nk = nk.replace("scale_shift_table", "modulation")
        out[nk] = v
    return out


def mm_to_diffusers(sd: StateDict) -> StateDict:
    out = {}
    for k, v in sd.items():
        if k == "head.modulation":
            out["scale_shift_table"] = v
            continue
        nk = k
        for a, b in _EXACT.items():
            if nk.startswith(b):
                nk = a + nk[len(b):]
                break
        else:
            for a, b in reversed(_SUBSTR):
                nk = nk.replace(b, a)
            if nk.startswith("blocks.") and nk.endswith(".modulation"):
                nk = nk[:-len("modulation")] + "scale_shift_table"
        out[nk] = v
    return out


def internal_ops():
    """MM names -> internal names (fused projections; conv patch embedding flattened)."""
    b = "blocks.{i}."
    ops = []
    for s in ("weight", "bias"):
        ops += [Merge([b + f"self_attn.proj_{x}.{s}" for x in "qkv"], b + f"self_attn.qkv.{s}"),
                Merge([b + f"cross_attn.proj_{x}.{s}" for x in "kv"], b + f"cross_attn.kv.{s}"),
                Merge([b + f"cross_attn.{x}_img.{s}" for x in "kv"], b + f"cross_attn.kv_img.{s}"),
                Rename(b + f"ffn.0.{s}", b + f"ffn_0.{s}"), Rename(b + f"ffn.2.{s}", b + f"ffn_2.{s}"),
                Rename(f"patch_embedding.{s}", f"embeddings.patch_embedding.{s}"),
                Rename(f"text_embedding.linear_1.{s}", f"embeddings.text_embedding_1.{s}"),
                Rename(f"text_embedding.linear_2.{s}", f"embeddings.text_embedding_2.{s}"),
                Rename(f"time_embedding.0.{s}", f"embeddings.time_embedding_0.{s}"),
                Rename(f"time_embedding.2.{s}", f"embeddings.time_embedding_2.{s}"),
                Rename(f"time_projection.1.{s}", f"embeddings.time_projection.{s}"),
                Rename(f"img_emb.proj.0.{s}", f"embeddings.img_emb_norm1.{s}"),
                Rename(f"img_emb.proj.1.{s}", f"embeddings.img_emb_fc1.{s}"),
                Rename(f"img_emb.proj.3.{s}", f"embeddings.img_emb_fc2.{s}"),
                Rename(f"img_emb.proj.4.{s}", f"embeddings.img_emb_norm2.{s}")]
    return ops


def mm_to_internal(sd: StateDict) -> StateDict:
    sd = dict(sd)
    w = sd.get("patch_embedding.weight")
    if w is not None and w.dim() == 5:
        sd["patch_embedding.weight"] = w.reshape(w.shape[0], -1)
    return apply_ops(sd, internal_ops())


def internal_to_mm(sd: StateDict, in_dim: int = 16, patch=(1, 2, 2)) -> StateDict:
    sd = revert_ops(dict(sd), internal_ops())
    w = sd.get("patch_embedding.weight")
    if w is not None and w.dim() == 2:
        sd["patch_embedding.weight"] = w.reshape(w.shape[0], in_dim, *patch)
    return sd
