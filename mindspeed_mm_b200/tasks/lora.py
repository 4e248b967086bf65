"""LoRA fine-tuning: low-rank adapters injected into the package's ``Linear`` layers before sharding.

``apply_lora(model, cfg)`` wraps every linear whose qualified name matches one of ``cfg.target_modules``
(exact suffix, or a ``{*}`` pattern) in a ``LoRALinear``: the base weight is frozen, ``lora_A`` [r, in]
(Kaiming-uniform) and ``lora_B`` [out, r] (zeros) are trainable and ``y = base(x) + (alpha / r) * (x A^T) B^T``.
Fused projections are targeted by their fused name or by any of their parts (``q_proj`` matches ``qkv_proj``), so
HF-style target lists keep working.  ``lora_state_dict`` / ``load_lora_state_dict`` give adapter-only
checkpoints and ``merge_lora`` folds adapters into the base weights.  Reference: PEFT injection before sharding,
wildcard matching and LoRA-only saving in mindspeed_mm/fsdp/utils/lora_utils.py:48-220 and lora_weight_manager.py:46;
Megatron-side wrapper mindspeed_mm/tasks/finetune/lora/lora_patch.py:54-365.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List

import torch
import torch.nn as nn

from .. import ops
from ..config.native import module_name_match
from ..models.qwen2_5_vl import Linear

_FUSED_PARTS = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj"),
                "attn_qkv": ("qkv",), "qkv": ("proj_q", "proj_k", "proj_v", "to_q", "to_k", "to_v"),
                "kv": ("proj_k", "proj_v")}


class LoRALinear(nn.Module):
    def __init__(self, base: Linear, rank: int, alpha: float, dropout: float = 0.0):
        super().__init__()
        self.base = base
        for p in base.parameters():
            p.requires_grad_(False)
        self.rank, self.scaling = rank, alpha / rank
        self.lora_A = nn.Parameter(torch.empty(rank, base.in_features))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, rank))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    @property
    def weight(self):          # code that reads ``layer.weight`` (fused epilogues) sees the frozen base weight
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def post_init(self):
        with torch.no_grad():
            bound = 1.0 / math.sqrt(self.lora_A.shape[1]) * math.sqrt(3.0)
            self.lora_A.uniform_(-bound, bound)
            self.lora_B.zero_()

    def forward(self, x):
        y = self.base(x)
        z = torch.nn.functional.linear(torch.nn.functional.linear(self.dropout(x), self.lora_A.to(x.dtype)), self.lora_B.to(x.dtype))
        return y + self.scaling * z


def _matches(name: str, targets: Iterable[str]) -> bool:
    leaf = name.rsplit(".", 1)[-1]
    for t in targets:
        if "{" in t and module_name_match(t, name):
            return True
        if name == t or name.endswith("." + t) or leaf == t:
            return True
        if any(t == part or t.endswith("." + part) for part in _FUSED_PARTS.get(leaf, ())):
            return True
    return False


def apply_lora(model: nn.Module, cfg) -> List[str]:
    """Wrap matching linears in place; freezes every other parameter.  Returns the wrapped module names."""
    targets = list(cfg.target_modules)
    wrapped = []
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if isinstance(child, Linear) and _matches(full, targets):
                setattr(mod, child_name, LoRALinear(child, cfg.rank, cfg.alpha, getattr(cfg, "dropout", 0.0)))
                wrapped.append(full)
    if not wrapped:
        raise ValueError(f"no module matched LoRA targets {targets}")
    for n, p in model.named_parameters():
        if "lora_A" not in n and "lora_B" not in n:
            p.requires_grad_(False)
    return wrapped


def lora_state_dict(named_full_params: Iterable) -> Dict[str, torch.Tensor]:
    return {n: t.detach().cpu().clone() for n, t in named_full_params if ".lora_A" in n or ".lora_B" in n}


def merge_lora(state: Dict[str, torch.Tensor], scaling: float) -> Dict[str, torch.Tensor]:
    """Fold ``B @ A * scaling`` into ``*.base.weight`` and drop the adapter tensors (keys lose ``.base``)."""
    out = {}
    for k, v in state.items():
        if ".lora_A" in k or ".lora_B" in k:
            continue
        if ".base." in k:
            stem = k.split(".base.")[0]
            nk = k.replace(".base.", ".")
            if k.endswith(".weight") and f"{stem}.lora_A" in state:
                v = v.float() + scaling * (state[f"{stem}.lora_B"].float() @ state[f"{stem}.lora_A"].float())
            out[nk] = v
        else:
            out[k] = v
    return out
