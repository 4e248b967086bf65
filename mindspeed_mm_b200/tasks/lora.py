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

    def forward(self, x, value_unused_in_backward: bool = False):
        y = self.base(x)                 # the adapter's sum needs the base value: never skipped in a recompute
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


# ------------------------------------------------------------------------------------------ PEFT adapter files
def to_peft_state(state: Dict[str, torch.Tensor], hf_ops) -> Dict[str, torch.Tensor]:
    """Adapter tensors under PEFT's names (``base_model.model.<hf module>.lora_A.weight`` / ``lora_B.weight``).

    ``state``: ``lora_state_dict`` output (internal names).  ``hf_ops``: the model's internal <-> Hugging Face operator list.
    An adapter on a fused projection (q|k|v, gate|up) is written as one adapter per Hugging Face part: every part gets the
    fused ``lora_A`` and its own rows of ``lora_B``, which is the same update."""
    from ..checkpoint import hf as hfio
    out: Dict[str, torch.Tensor] = {}
    for k, b in state.items():
        if not k.endswith(".lora_B"):
            continue
        stem = k[:-len(".lora_B")]
        a = state[stem + ".lora_A"]
        parts = hfio.to_hf({stem + ".weight": b.clone()}, hf_ops)          # rows of B follow the rows of the weight
        for name, bp in parts.items():
            mod = name[:-len(".weight")]
            out[f"base_model.model.{mod}.lora_A.weight"] = a.clone()
            out[f"base_model.model.{mod}.lora_B.weight"] = bp.contiguous()
    return out


def save_peft_adapter(state: Dict[str, torch.Tensor], hf_ops, out_dir: str, cfg, base_model: str = "") -> None:
    """``adapter_model.safetensors`` + ``adapter_config.json`` as PEFT writes them (the reference's LoRA-only saving,
    mindspeed_mm/fsdp/utils/lora_weight_manager.py:46)."""
    import json
    import os
    from safetensors.torch import save_file
    os.makedirs(out_dir, exist_ok=True)
    peft = to_peft_state(state, hf_ops)
    save_file(peft, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
    targets = sorted({k.split(".")[-3] for k in peft})
    with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
        json.dump({"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": int(cfg.rank), "lora_alpha": float(cfg.alpha),
                   "lora_dropout": float(getattr(cfg, "dropout", 0.0)), "target_modules": targets, "bias": "none",
                   "fan_in_fan_out": False, "inference_mode": True, "base_model_name_or_path": base_model}, f, indent=1)


def from_peft_state(peft: Dict[str, torch.Tensor], hf_ops) -> Dict[str, torch.Tensor]:
    """Inverse of ``to_peft_state``.  Parts of a fused projection must share ``lora_A`` (as adapters written by
    ``save_peft_adapter`` do); independently trained part adapters would need a fused rank of the parts' sum and are
    refused with the reason."""
    from ..checkpoint import hf as hfio
    pre = "base_model.model."
    b_hf = {k[len(pre):-len(".lora_B.weight")] + ".weight": v for k, v in peft.items() if k.endswith(".lora_B.weight")}
    a_hf = {k[len(pre):-len(".lora_A.weight")] + ".weight": v for k, v in peft.items() if k.endswith(".lora_A.weight")}
    internal_b = hfio.to_internal(b_hf, hf_ops)
    internal_a = hfio.to_internal(a_hf, hf_ops)        # the same renames / merges: fused modules get their parts' A stacked
    out: Dict[str, torch.Tensor] = {}
    for name, b in internal_b.items():
        stem, r = name[:-len(".weight")], b.shape[1]
        parts = internal_a[name].split(r, dim=0)
        if any(not torch.equal(parts[0], p) for p in parts[1:]):
            raise NotImplementedError(f"{stem}: its {len(parts)} Hugging Face parts carry different lora_A; a fused adapter "
                                      f"of rank {r * len(parts)} would be needed")
        out[stem + ".lora_A"], out[stem + ".lora_B"] = parts[0].clone(), b
    return out
