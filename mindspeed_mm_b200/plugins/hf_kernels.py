"""Kernel substitution for Hugging Face ``transformers`` model classes.

``apply_kernel_plugin()`` swaps the hot element-wise and attention paths of the stock Qwen2 / Qwen2.5-VL / Qwen3 /
Qwen3-MoE / Qwen3-VL(-MoE) modeling files for this package's ops, so that code that builds those classes itself
(an RL trainer such as verl, an evaluation harness, ``runtime/trainer.py`` with ``model_id: hf_auto``) runs on the sm_100a
kernels without a change on its side.  Reference: verl_plugin/verl_npu/plugin.py:33-159 (``apply_npu_plugin``: RMSNorm,
rotary embedding, SwiGLU MLP and fused MoE experts replaced on the transformers classes at import time) and
mindspeed_mm/fsdp/ops/flash_attn/flash_attn.py (attention registered through the transformers attention interface).

What is replaced, per modeling module:

* ``*RMSNorm.forward``                     -> ``ops.rms_norm``
* ``*MLP.forward`` (gate / up / down, SiLU) -> ``down(ops.swiglu([gate(x) | up(x)]))``
* ``apply_rotary_pos_emb``                 -> ``ops.rope_rotate_half`` on the token-major view
* attention implementation ``"mm_b200"``   -> ``ops.attention_varlen`` (packed batches through the flash-attention
  keyword arguments ``cu_seq_lens_q`` / ``cu_seq_lens_k``) or ``ops.attention_dense`` (no padding mask); a batch with
  padding falls back to ``scaled_dot_product_attention`` with the mask it was given
* fused experts with the ``[E, H, 2F]`` / ``[E, F, H]`` parameter layout (transformers < 5) -> grouped GEMM

Every replacement keeps the signature of what it replaces; ``remove_kernel_plugin()`` restores the originals.  On a CPU
tensor the ops run their PyTorch reference, so the patched classes stay usable everywhere.
"""
from __future__ import annotations

import importlib
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops

DEFAULT_MODULES = ("qwen2", "qwen2_vl", "qwen2_5_vl", "qwen3", "qwen3_moe", "qwen3_vl", "qwen3_vl_moe", "qwen3_5",
                   "qwen3_5_moe", "internvl", "llama", "mistral")
ATTENTION_NAME = "mm_b200"
# Same function under a name that contains "flash": vision and audio towers of transformers hand their window / image
# boundaries (``cu_seq_lens_q``) to the attention function only when the implementation's name says so, and otherwise loop
# over the windows one call at a time.
TOWER_ATTENTION_NAME = "mm_b200_flash"

_saved: List[Tuple[object, str, object]] = []        # (owner, attribute, original) for remove_kernel_plugin


def _set(owner, name: str, value) -> None:
    _saved.append((owner, name, getattr(owner, name)))
    setattr(owner, name, value)


# ------------------------------------------------------------------------------------------------ replacements
def _rms_norm_forward(self, hidden_states):
    eps = getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6))
    return ops.rms_norm(hidden_states, self.weight.to(hidden_states.dtype), eps)


def _swiglu_mlp_forward(self, x):
    if not isinstance(self.act_fn, nn.SiLU) and getattr(self.act_fn, "__name__", "") != "silu" \
            and type(self.act_fn).__name__ not in ("SiLUActivation", "SiLU"):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))      # another gate activation
    gate_up = torch.cat((self.gate_proj(x), self.up_proj(x)), dim=-1)
    return self.down_proj(ops.swiglu(gate_up))


def _rotary(q, k, cos, sin, position_ids=None, unsqueeze_dim: int = 1):
    """q, k: [B, heads, S, D] (``unsqueeze_dim`` 1) or [B, S, heads, D] (2); cos, sin: [B, S, D]."""
    def one(x):
        xt = x.transpose(1, 2) if unsqueeze_dim == 1 else x                    # [B, S, heads, D]
        B, S, N, D = xt.shape
        c, s = cos.expand(B, S, D).reshape(B * S, D), sin.expand(B, S, D).reshape(B * S, D)
        y = ops.rope_rotate_half(xt.reshape(B * S, N, D), c.to(x.dtype), s.to(x.dtype)).view(B, S, N, D)
        return y.transpose(1, 2) if unsqueeze_dim == 1 else y
    return one(q), one(k)


def attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0, scaling: Optional[float] = None,
                      is_causal: Optional[bool] = None, **kwargs):
    """transformers attention-interface entry: query [B, Hq, Sq, D], key / value [B, Hkv, Sk, D] -> ([B, Sq, Hq, D], None)."""
    B, Hq, Sq, D = query.shape
    Sk = key.shape[2]
    causal = bool(is_causal if is_causal is not None else getattr(module, "is_causal", True)) and Sq > 1
    q, k, v = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    cu_q, cu_k = kwargs.get("cu_seq_lens_q"), kwargs.get("cu_seq_lens_k")
    if cu_q is not None and cu_k is not None and B == 1:
        o = ops.attention_varlen(q[0].contiguous(), k[0].contiguous(), v[0].contiguous(), cu_q.to(torch.int32),
                                 cu_k.to(torch.int32), int(kwargs.get("max_length_q", Sq)),
                                 int(kwargs.get("max_length_k", Sk)), causal=causal, softmax_scale=scaling)
        return o[None], None
    if attention_mask is None and (not causal or Sq == Sk):
        return ops.attention_dense(q.contiguous(), k.contiguous(), v.contiguous(), causal=causal, softmax_scale=scaling), None
    # padding (2-D mask), a key / value cache (Sq != Sk) or a custom 4-D mask: the library kernel with that mask
    mask = attention_mask
    if mask is not None and mask.dim() == 2:
        keep = mask[:, None, None, :Sk].bool()
        if causal:
            keep = keep & torch.ones(Sq, Sk, dtype=torch.bool, device=query.device).tril(Sk - Sq)
        mask = keep
    elif mask is None and causal:
        mask = torch.ones(Sq, Sk, dtype=torch.bool, device=query.device).tril(Sk - Sq)
    rep = Hq // key.shape[1]
    if rep > 1:
        key, value = key.repeat_interleave(rep, 1), value.repeat_interleave(rep, 1)
    o = F.scaled_dot_product_attention(query, key, value, attn_mask=mask, dropout_p=0.0, scale=scaling)
    return o.transpose(1, 2).contiguous(), None


class _GroupedExperts:
    """forward of a fused-experts module whose parameters are ``gate_up_proj [E, H, 2F]`` and ``down_proj [E, F, H]``."""

    @staticmethod
    def forward(self, hidden_states, routing_weights, router_indices):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        if routing_weights.shape[-1] != router_indices.shape[-1]:                # dense [T, E] table: pick the top-k entries
            routing_weights = routing_weights.gather(1, router_indices)
        out = ops.moe_experts(x, router_indices, routing_weights.to(x.dtype), self.gate_up_proj, self.down_proj)
        return out.view(shape)


# ------------------------------------------------------------------------------------------------ apply / remove
def _patch_module(mod, record: Dict[str, List[str]]) -> None:
    done = record.setdefault(mod.__name__.rsplit(".", 1)[-1], [])
    for name, obj in list(vars(mod).items()):
        if not isinstance(obj, type) or not issubclass(obj, nn.Module) or obj.__module__ != mod.__name__:
            continue
        if name.endswith("RMSNorm") and "Gated" not in name and "forward" in vars(obj) and _plain_rms(obj):
            _set(obj, "forward", _rms_norm_forward)
            done.append(name)
        elif name.endswith("MLP") and _is_swiglu_mlp(obj):
            _set(obj, "forward", _swiglu_mlp_forward)
            done.append(name)
        elif name.endswith("Experts") and _is_fused_experts(obj) and hasattr(ops, "moe_experts"):
            _set(obj, "forward", _GroupedExperts.forward)
            done.append(name)
    if "apply_rotary_pos_emb" in vars(mod) and _rotary_signature_ok(mod.apply_rotary_pos_emb):
        _set(mod, "apply_rotary_pos_emb", _rotary)
        done.append("apply_rotary_pos_emb")


def _plain_rms(cls) -> bool:
    """``weight * normalised(x)``: classes that add 1 to the weight (Gemma, Qwen3.5) or gate the output keep their own."""
    import inspect
    try:
        src = inspect.getsource(cls.forward)
    except (OSError, TypeError):
        return False
    return "1.0 +" not in src and "1 +" not in src and "gate" not in src


def _is_swiglu_mlp(cls) -> bool:
    import inspect
    try:
        src = inspect.getsource(cls)
    except (OSError, TypeError):
        return False
    return all(s in src for s in ("gate_proj", "up_proj", "down_proj")) and "self.act_fn(self.gate_proj(" in src \
        and "bias=True" not in src


def _is_fused_experts(cls) -> bool:
    import inspect
    try:
        src = inspect.getsource(cls.__init__)
    except (OSError, TypeError):
        return False
    return "self.hidden_size, 2 * self.expert_dim" in src.replace("\n", " ")


def _rotary_signature_ok(fn) -> bool:
    import inspect
    names = list(inspect.signature(fn).parameters)
    return names[:4] == ["q", "k", "cos", "sin"] and "mrope_section" not in names


def apply_kernel_plugin(modules: Sequence[str] = DEFAULT_MODULES, attention: bool = True) -> Dict[str, List[str]]:
    """Patch the listed ``transformers.models.<name>.modeling_<name>`` modules (missing ones are skipped) and register
    the ``"mm_b200"`` attention implementation.  Returns ``{module: [patched names]}``."""
    if _saved:
        remove_kernel_plugin()
    record: Dict[str, List[str]] = {}
    for name in modules:
        try:
            mod = importlib.import_module(f"transformers.models.{name}.modeling_{name}")
        except Exception:                    # a family this transformers version does not ship
            continue
        _patch_module(mod, record)
    if attention:
        from transformers import AttentionInterface, AttentionMaskInterface
        from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
        # same mask contract as flash attention: no mask without padding, the 2-D padding mask otherwise
        for name in (ATTENTION_NAME, TOWER_ATTENTION_NAME):
            AttentionInterface.register(name, attention_forward)
            AttentionMaskInterface.register(name, ALL_MASK_ATTENTION_FUNCTIONS["flash_attention_2"])
        record["attention"] = [ATTENTION_NAME, TOWER_ATTENTION_NAME]
    return record


def remove_kernel_plugin() -> None:
    while _saved:
        owner, name, orig = _saved.pop()
        setattr(owner, name, orig)


def use_plugin_attention(model_or_config, packed_towers: bool = False) -> None:
    """Select the registered attention implementation on a config or an already built model (all sub-configs).
    ``packed_towers``: vision / audio towers go under the flash-named alias so that they take their packed (varlen) path
    instead of one call per window.  Off by default: that path is verified on CPU only (on a B200 the stock Qwen2.5-VL
    tower failed under it), so towers keep the per-window calls unless asked."""
    cfg = getattr(model_or_config, "config", model_or_config)
    for n in (None, "text_config", "vision_config", "audio_config"):
        c = cfg if n is None else getattr(cfg, n, None)
        if c is not None:
            c._attn_implementation = TOWER_ATTENTION_NAME if packed_towers and n in ("vision_config", "audio_config") \
                else ATTENTION_NAME
