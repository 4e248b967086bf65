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


def _build_kl_family(mid: str, block: dict):
    """The KL / VQ autoencoders other than Wan's (``models/ae/kl_vae.py``), selected by the reference's ``model_id``s."""
    from .ae import kl_vae as K
    mid = mid.lower()
    cfg_keys = {k: block[k] for k in ("in_channels", "out_channels", "base", "ch_mult", "num_res_blocks", "z_channels",
                                      "temporal_down", "kt", "mid_attention", "scale_factor", "shift_factor") if k in block}
    if "ch" in block:
        cfg_keys.setdefault("base", block["ch"])
    tiling = {k: block[k] for k in ("tile_sample_min", "tile_overlap", "tile_frames") if k in block}
    if mid in ("flux_vae", "fluxvae"):
        return K.AutoencoderKL2D(K.KLVAEConfig.flux(**{k: v for k, v in cfg_keys.items() if k not in ("z_channels", "scale_factor", "shift_factor", "kt")}))
    if mid in ("vae", "autoencoderkl", "autoencoder_kl", "diffusers_ae", "sd3_vae", "sd_vae"):
        preset = K.KLVAEConfig.sd3 if "sd3" in mid or block.get("z_channels", 16) == 16 else K.KLVAEConfig.sd
        base = preset()
        for k, v in cfg_keys.items():
            setattr(base, k, tuple(v) if isinstance(v, list) else v)
        base.kt = 1
        return K.AutoencoderKL2D(base)
    if mid in ("casualvae", "causalvae", "contextparallelcasualvae", "autoencoder_kl_hunyuanvideo", "hunyuanvideo_vae",
               "hunyuanvideo_15_vae", "stepvideovae", "stepvideo_vae", "vae3d", "vae_temporal"):
        preset = K.KLVAEConfig.hunyuan_video if "hunyuan" in mid else K.KLVAEConfig.open_sora_plan
        base = preset()
        for k, v in cfg_keys.items():
            setattr(base, k, tuple(v) if isinstance(v, list) else v)
        vae = K.CausalVAE3D(base, **tiling)
        vae.enable_tiling(bool(block.get("use_tiling", block.get("enable_tiling", False))))
        return vae
    if mid in ("wfvae", "wf_vae"):
        return K.WFVAE(**{k: block[k] for k in ("base", "z_channels", "in_channels", "num_res_blocks", "energy_flow", "scale_factor",
                                                "shift_factor", "mid_attention") if k in block})
    if mid in ("movq", "movqvae"):
        return K.MOVQ(**{k: block[k] for k in ("z_channels", "in_channels", "base", "ch_mult", "num_res_blocks", "n_embed",
                                               "embed_dim", "mid_attention") if k in block})
    return None


def build_ae(block: Optional[dict], device="cpu", dtype=torch.float32):
    if not block:
        return None
    mid = block.get("model_id", "wan_video_vae")
    if mid not in ("wan_video_vae", "wan_vae", "autoencoder_kl_wan"):
        vae = _build_kl_family(mid, block)
        if vae is None:
            from .registry import build_model
            return build_model(mid, block)
        src = block.get("from_pretrained")
        if src and os.path.exists(src):
            vae.load_state_dict(_load_safetensors_dir(src), strict=False)
        return vae.to(device=device, dtype=dtype).eval().requires_grad_(False)
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
    if "glyph" in mid or "byt5" in mid:
        # byte-level T5 over the quoted spans of the prompt (mindspeed_mm/models/text_encoder/hunyuan15_glyph_text_encoder.py)
        from .prompt_encoders import ByteTokenizer, GlyphByT5Encoder, GlyphEncoderConfig
        from .registry import config_from_dict
        cfg = config_from_dict(GlyphEncoderConfig, {k: v for k, v in block.items() if k not in ("model_id", "from_pretrained")})
        return GlyphByT5Encoder(cfg, ByteTokenizer())
    if "stepllm" in mid or "step_llm" in mid:
        from .prompt_encoders import StepLLMConfig, StepLLMEncoder
        from .registry import config_from_dict
        return StepLLMEncoder(config_from_dict(StepLLMConfig, {k: v for k, v in block.items() if k not in ("model_id", "from_pretrained")}))
    if "mllm" in mid:
        # decoder-only LM read at an inner layer behind an instruction template
        # (mindspeed_mm/models/text_encoder/hunyuan15_mllm_text_encoder.py:63-121)
        from .prompt_encoders import TEMPLATES, DecoderPromptEncoder
        from .registry import build_model
        lm = build_model(block.get("lm_model_id", "llava"), block.get("lm_config"))
        tpl = block.get("template") or TEMPLATES.get(block.get("template_id", "encode-video"))
        return DecoderPromptEncoder(lm, tpl, int(block.get("hidden_state_skip_layer", 2)), bool(block.get("apply_final_norm", False)))
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
