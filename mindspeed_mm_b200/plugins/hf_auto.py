"""``model_id: hf_auto``: train whatever architecture a Hugging Face ``config.json`` names, built from the stock
``transformers`` class on the meta device and run under the ZeRO-3 engine (``hf_adapter.HFModelAdapter``) with this
package's kernels substituted into it (``hf_kernels.apply_kernel_plugin``).

Reference: mindspeed_mm/fsdp/models/modelhub.py:60-70 (``AutoConfig`` -> model class -> ``init_model_with_meta_device``)
and the per-family wrappers under mindspeed_mm/models/transformers/ that register stock classes with the trainer.
The recipe either points ``model.model_name_or_path`` at a checkpoint directory (its ``config.json`` is read, its
weights are loaded by name) or carries the Hugging Face config inline under ``model.config.hf``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch.nn as nn

from ..models.registry import model_register
from .hf_adapter import HFModelAdapter


@dataclass
class HFAutoConfig:
    hf: dict = field(default_factory=dict)          # the Hugging Face config as a dict (``model_type`` required)
    model_class: Optional[str] = None               # a ``transformers`` class name; default: chosen from the config
    kernel_plugin: bool = True                      # substitute this package's ops into the modeling module
    attn_implementation: Optional[str] = None       # default: "mm_b200" with the plugin, else "sdpa"
    unit_classes: Optional[tuple] = None            # sharding units; default: the model's ``_no_split_modules``
    init_std: float = 0.02

    @staticmethod
    def from_hf(hf: dict) -> "HFAutoConfig":
        return HFAutoConfig(hf=dict(hf))

    def build_hf_config(self):
        from transformers import AutoConfig
        if "model_type" not in self.hf:
            raise ValueError("hf_auto needs a Hugging Face config with a model_type (model.model_name_or_path/config.json "
                             "or model.config.hf)")
        kw = {k: v for k, v in self.hf.items() if k not in ("model_type", "architectures", "transformers_version")}
        return AutoConfig.for_model(self.hf["model_type"], **kw)


class _ConfigView:
    """The Hugging Face config seen through the attribute names the data builders read on native configs (``text``,
    ``vision``); everything else is the Hugging Face config's own attribute."""

    def __init__(self, hf_cfg):
        self._hf = hf_cfg

    @property
    def text(self):
        return self._hf.get_text_config() if hasattr(self._hf, "get_text_config") else self._hf

    @property
    def vision(self):
        return getattr(self._hf, "vision_config", None)

    @property
    def image_token_id(self):
        hf = self._hf
        for n in ("image_token_id", "image_token_index"):
            if getattr(hf, n, None) is not None:
                return getattr(hf, n)
        return self.text.vocab_size - 1

    @property
    def vision_start_token_id(self):
        v = getattr(self._hf, "vision_start_token_id", None)
        return v if v is not None else self.image_token_id

    def __getattr__(self, name):
        return getattr(self._hf, name)


@model_register.register("hf_auto")
class HFAutoModel(HFModelAdapter):
    config_class = HFAutoConfig

    def __init__(self, config: HFAutoConfig, **_):
        import transformers
        hf_cfg = config.build_hf_config()
        if config.kernel_plugin:
            from . import hf_kernels
            hf_kernels.apply_kernel_plugin()
        hf_cfg._attn_implementation = config.attn_implementation or ("mm_b200" if config.kernel_plugin else "sdpa")
        for sub in ("text_config", "vision_config", "audio_config"):
            if getattr(hf_cfg, sub, None) is not None:
                getattr(hf_cfg, sub)._attn_implementation = hf_cfg._attn_implementation
        if config.model_class:
            cls = getattr(transformers, config.model_class)
            model = cls(hf_cfg)
        else:
            auto = transformers.AutoModelForImageTextToText if getattr(hf_cfg, "vision_config", None) is not None \
                else transformers.AutoModelForCausalLM
            model = auto.from_config(hf_cfg)
        super().__init__(model, unit_classes=config.unit_classes)
        self._param_names = [n for n, _ in model.named_parameters()]
        self.auto_config = config
        self.hf_config = hf_cfg
        self.config = _ConfigView(hf_cfg)
        self.init_std = config.init_std

    def hf_ops(self):
        from ..checkpoint.hf import MatchBySuffix, UnderPrefix
        from ..checkpoint.operators import Operator
        ops = [MatchBySuffix(self._param_names)]
        tied = getattr(self.model, "_untied_head", None)
        if tied is not None:
            emb, head = tied

            class _FillHead(Operator):
                exact_names = True

                def apply(self, sd):
                    if head not in sd and emb in sd:
                        sd[head] = sd[emb].clone()

                def revert(self, sd):
                    pass
            ops.append(_FillHead())
        return ops + [UnderPrefix("model.")]
