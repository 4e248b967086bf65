"""Builds the frozen conditioning towers of a generative model from its ``ae`` / ``text_encoder`` config blocks.

Config shape follows the reference's model json (examples/wan2.1/*/pretrain_model.json): ``ae.model_id`` with
``from_pretrained``; ``text_encoder`` as a block or a list of blocks with ``model_id`` / ``hub_backend`` /
``from_pretrained``.  Weights are read from ``*.safetensors`` files in ``from_pretrained`` when that directory
exists; otherwise the tower keeps its random initialisation (synthetic-data runs).
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Optional

import torch


def _load_safetensors_dir(path: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    sd: Dict[str, torch.Tensor] = {}
    files = [path] if os.path.isfile(path) else sorted(glob.glob(os.path.join(path, "*.safetensors")))
    for f in files:
        sd.update(load_file(f))
    return sd


def build_ae(block: Optional[dict], device="cpu", dtype=torch.float32):
    if not block:
        return None
    mid = block.get("model_id", "wan_video_vae")
    if mid not in ("wan_video_vae", "wan_vae", "autoencoder_kl_wan"):
        from .registry import build_model
        return build_model(mid, block)
    from .ae.wan_vae import WanVAE, WanVAEConfig
    keys = {k: block[k] for k in ("base_dim", "z_dim", "dim_mult", "num_res_blocks", "attn_scales", "temporal_downsample",
                                  "latents_mean", "latents_std") if k in block}
    vae = WanVAE(WanVAEConfig(**keys))
    src = block.get("from_pretrained")
    if src and os.path.exists(src):
        vae.load_state_dict(_load_safetensors_dir(src), strict=False)
    return vae.to(device=device, dtype=dtype).eval().requires_grad_(False)


def _one_text_encoder(block: dict):
    from .text_encoder import CLIPTextConfig, CLIPTextEncoder, T5Config, T5Encoder
    mid = str(block.get("model_id", "UMT5")).lower()
    src = block.get("from_pretrained")
    have = bool(src) and os.path.exists(src)
    if "t5" in mid:
        cfg = T5Config(**{k: block[k] for k in ("vocab_size", "d_model", "d_kv", "d_ff", "num_layers", "num_heads",
                                                "num_buckets", "max_distance") if k in block},
                       per_layer_bias="umt5" in mid or block.get("per_layer_bias", False),
                       gated=block.get("gated", True))
        enc = T5Encoder(cfg)
        if have:
            enc.load_hf_state_dict(_load_safetensors_dir(src))
        return enc
    if "clip" in mid:
        cfg = CLIPTextConfig(**{k: block[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_layers",
                                                      "num_heads", "max_positions", "eos_token_id", "act") if k in block})
        enc = CLIPTextEncoder(cfg)
        if have:
            enc.load_hf_state_dict(_load_safetensors_dir(src))
        return enc
    from .registry import build_model
    return build_model(block["model_id"], block)


def build_text_encoder(block, device="cpu", dtype=torch.float32):
    if not block:
        return None
    from .text_encoder import TextEncoder
    encs = [_one_text_encoder(b) for b in block] if isinstance(block, (list, tuple)) else _one_text_encoder(block)
    return TextEncoder(encs).to(device=device, dtype=dtype).eval()
