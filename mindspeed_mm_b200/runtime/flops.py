"""Model FLOPs accounting for MFU reports (the reference's flops_tool: mindspeed_mm/fsdp/tools/flops_tool/*.py).

Counts the matmul FLOPs of one forward pass (2 * M * N * K per GEMM, attention as 4 * S_q * S_k * D per head,
halved for causal); a training step with full recompute is 4x forward, without recompute 3x.
"""
from __future__ import annotations

from typing import Sequence


def qwen25vl_forward_flops(cfg, text_seqlens: Sequence[int], vision_tokens: int, window_tokens: int = 64) -> float:
    t, v = cfg.text, cfg.vision
    T = sum(text_seqlens)
    hd = t.head_dim
    per_layer = 2 * T * t.hidden_size * ((t.num_attention_heads + 2 * t.num_key_value_heads) * hd
                                         + t.num_attention_heads * hd + 3 * t.intermediate_size)
    attn = sum(4 * s * s * hd * t.num_attention_heads * 0.5 for s in text_seqlens)
    llm = t.num_layers * (per_layer + attn) + 2 * T * t.hidden_size * t.vocab_size
    ffn = (v.intermediate_size + 63) // 64 * 64
    vit_layer = 2 * vision_tokens * v.hidden_size * (4 * v.hidden_size + 3 * ffn)
    vd = v.hidden_size // v.num_heads
    n_full = len(v.fullatt_block_indexes)
    per_img = vision_tokens  # upper bound when all tokens belong to one image
    vit_attn = (v.depth - n_full) * 4 * vision_tokens * window_tokens * vd * v.num_heads + n_full * 4 * vision_tokens * per_img * vd * v.num_heads
    m = v.hidden_size * v.spatial_merge_size ** 2
    merger = 2 * (vision_tokens // v.spatial_merge_size ** 2) * (m * m + m * v.out_hidden_size)
    return float(llm + v.depth * vit_layer + vit_attn + merger)


def wan_forward_flops(cfg, tokens: int, text_len: int, batch: int = 1) -> float:
    H, F = cfg.hidden_size, cfg.ffn_dim
    per = 2 * tokens * H * (3 * H + H) + 4 * tokens * tokens * H          # self attention
    per += 2 * tokens * H * 2 * H + 2 * text_len * H * 2 * H + 4 * tokens * text_len * H   # cross attention
    per += 2 * tokens * H * 2 * F
    return float(batch * cfg.num_layers * per)


def training_flops(forward_flops: float, recompute: bool = True) -> float:
    return forward_flops * (4.0 if recompute else 3.0)


def mfu(step_flops: float, step_seconds: float, n_gpus: int, peak_tflops: float) -> float:
    return step_flops / step_seconds / (n_gpus * peak_tflops * 1e12)
