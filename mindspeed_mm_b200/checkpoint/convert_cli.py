"""``mm-convert <Converter> <command> [--cfg.a.b value ...]`` - offline checkpoint conversion (CPU, one process).

Command surface of the reference's CLI (checkpoint/convert_cli.py:13, checkpoint/common/converter.py:8-50):

    mm-convert Qwen2_5_VLConverter hf_to_mm --cfg.mm_dir OUT --cfg.hf_config.hf_dir HF \
        --cfg.parallel_config.llm_pp_layers [[12,16]] --cfg.parallel_config.vit_pp_layers [[32,0]] \
        --cfg.parallel_config.tp_size 2
    mm-convert Qwen2_5_VLConverter mm_to_hf --cfg.save_hf_dir OUT --cfg.mm_dir MM --cfg.hf_config.hf_dir HF ...
    mm-convert Qwen2_5_VLConverter resplit  --cfg.source_dir MM --cfg.target_dir OUT --cfg.source_parallel_config.* --cfg.target_parallel_config.*
    mm-convert Qwen2_5_VLConverter hf_to_dcp --cfg.hf_dir HF --cfg.dcp_dir OUT
    mm-convert Qwen2_5_VLConverter dcp_to_hf --cfg.hf_dir HF --cfg.dcp_dir IN --cfg.save_hf_dir OUT
    mm-convert WanConverter hf_to_mm|mm_to_hf --cfg.source_path IN --cfg.target_path OUT

Dotted ``--cfg.*`` options are collected into a nested dict (values parsed as YAML, so lists work).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Any, Dict, List

import torch
import yaml

from . import hf as hfio
from . import megatron as mm

CONVERTERS: Dict[str, type] = {}


def register(cls):
    CONVERTERS[cls.__name__] = cls
    return cls


def parse_cfg(argv: List[str]) -> Dict[str, Any]:
    cfg: Dict[str, Any] = {}
    i = 0
    while i < len(argv):
        tok = argv[i]
        if not tok.startswith("--"):
            raise SystemExit(f"unexpected argument {tok!r}")
        key, eq, val = tok[2:].partition("=")
        if not eq:
            i += 1
            if i >= len(argv):
                raise SystemExit(f"missing value for --{key}")
            val = argv[i]
        parts = key.split(".")
        if parts[0] == "cfg":
            parts = parts[1:]
        node = cfg
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = yaml.safe_load(val)
        i += 1
    return cfg


def _flat_layers(x) -> List[int]:
    """``[[12,16]]`` (virtual-pipeline outer list) or ``[12,16]`` -> ``[12,16]``."""
    if x and isinstance(x[0], (list, tuple)):
        if len(x) != 1:
            raise NotImplementedError("virtual pipeline chunks (>1 outer list) are written as model0/model1 keys; "
                                      "use one chunk per stage here")
        return list(x[0])
    return list(x)


def _hf_model_config(hf_dir: str) -> dict:
    with open(os.path.join(hf_dir, "config.json")) as f:
        c = json.load(f)
    t = c.get("text_config", c)
    v = c["vision_config"]
    nh = t["num_attention_heads"]
    return dict(num_heads=nh, num_kv_heads=t.get("num_key_value_heads", nh),
                head_dim=t.get("head_dim") or t["hidden_size"] // nh, vit_heads=v["num_heads"],
                llm_layers=t["num_hidden_layers"], vit_layers=v["depth"])


class _VLMConverter:
    glu_vit = True

    @classmethod
    def _ops(cls, m):
        return mm.qwen25vl_mm_ops(m["num_heads"], m["num_kv_heads"], m["head_dim"], m["vit_heads"], cls.glu_vit)

    @classmethod
    def hf_to_mm(cls, cfg):
        hf_dir = cfg["hf_config"]["hf_dir"]
        m = _hf_model_config(hf_dir)
        pc = cfg.get("parallel_config", {})
        llm = _flat_layers(pc.get("llm_pp_layers", [[m["llm_layers"]]]))
        vit = _flat_layers(pc.get("vit_pp_layers", [[m["vit_layers"]] + [0] * (len(llm) - 1)]))
        if sum(llm) != m["llm_layers"] or sum(vit) != m["vit_layers"] or len(llm) != len(vit):
            raise SystemExit(f"pp layer lists {vit} / {llm} do not add up to {m['vit_layers']} / {m['llm_layers']}")
        sds = mm.hf_to_mm(hfio.load_state_dict(hf_dir), cls._ops(m), int(pc.get("tp_size", 1)), vit, llm, cls.glu_vit)
        mm.save_mm(sds, cfg["mm_dir"])

    @classmethod
    def mm_to_hf(cls, cfg):
        hf_dir = cfg["hf_config"]["hf_dir"]
        m = _hf_model_config(hf_dir)
        pc = cfg.get("parallel_config", {})
        llm = _flat_layers(pc.get("llm_pp_layers", [[m["llm_layers"]]]))
        vit = _flat_layers(pc.get("vit_pp_layers", [[m["vit_layers"]] + [0] * (len(llm) - 1)]))
        sd = mm.mm_to_hf(mm.load_mm(cfg["mm_dir"]), cls._ops(m), vit, llm, cls.glu_vit)
        hfio.save_sharded(sd, cfg["save_hf_dir"])
        for f in os.listdir(hf_dir):
            if f.endswith((".json", ".txt", ".jinja")) and f != hfio.INDEX:
                import shutil
                shutil.copy(os.path.join(hf_dir, f), os.path.join(cfg["save_hf_dir"], f))

    @classmethod
    def resplit(cls, cfg):
        m = _hf_model_config(cfg["hf_config"]["hf_dir"]) if "hf_config" in cfg else cfg["model"]
        s, t = cfg["source_parallel_config"], cfg["target_parallel_config"]
        ops = cls._ops(m)
        sd = mm.mm_to_hf(mm.load_mm(cfg["source_dir"]), ops, _flat_layers(s["vit_pp_layers"]),
                         _flat_layers(s["llm_pp_layers"]), cls.glu_vit, modern_prefix=False)
        out = mm.hf_to_mm(sd, cls._ops(m), int(t.get("tp_size", 1)), _flat_layers(t["vit_pp_layers"]),
                          _flat_layers(t["llm_pp_layers"]), cls.glu_vit)
        mm.save_mm(out, cfg["target_dir"])

    @staticmethod
    def hf_to_dcp(cfg):
        import torch.distributed.checkpoint as dcp
        sd = hfio.load_state_dict(cfg["hf_dir"])
        dcp.save({"model": sd}, checkpoint_id=os.path.join(cfg["dcp_dir"], "release"), no_dist=True)
        with open(os.path.join(cfg["dcp_dir"], "latest_checkpointed_iteration.txt"), "w") as f:
            f.write("release")

    @staticmethod
    def dcp_to_hf(cfg):
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.format_utils import dcp_to_torch_save
        src = cfg["dcp_dir"]
        tr = os.path.join(src, "latest_checkpointed_iteration.txt")
        if os.path.exists(tr):
            tag = open(tr).read().strip()
            src = os.path.join(src, tag if tag == "release" else f"iter_{int(tag):07d}")
        tmp = os.path.join(cfg["save_hf_dir"], "_dcp_tmp.pt")
        os.makedirs(cfg["save_hf_dir"], exist_ok=True)
        dcp_to_torch_save(src, tmp)
        sd = torch.load(tmp, map_location="cpu", weights_only=False)
        os.remove(tmp)
        sd = sd.get("model", sd)
        hfio.save_sharded({k: v for k, v in sd.items() if isinstance(v, torch.Tensor)}, cfg["save_hf_dir"])


@register
class Qwen2_5_VLConverter(_VLMConverter):
    glu_vit = True


@register
class Qwen2VLConverter(_VLMConverter):
    glu_vit = False


@register
class WanConverter:
    @staticmethod
    def hf_to_mm(cfg):
        from .wan import diffusers_to_mm
        hfio.save_sharded(diffusers_to_mm(hfio.load_state_dict(cfg["source_path"])), cfg["target_path"])

    @staticmethod
    def mm_to_hf(cfg):
        from .wan import mm_to_diffusers
        hfio.save_sharded(mm_to_diffusers(hfio.load_state_dict(cfg["source_path"])), cfg["target_path"])


class _DcpHFConverter:
    """``hf_to_dcp`` / ``dcp_to_hf`` in the layout the reference's native trainer reads and writes for the Qwen3 families
    (checkpoint/vlm_model/converters/qwen3vl.py:36-118): every key gets the ``model.`` prefix of the wrapped module and the
    fused expert tensors ``[E, in, out]`` are stored as 2-D ``[E * in, out]``."""
    fused_linear_names = ("mlp.experts.gate_up_proj", "mlp.experts.down_proj")
    dcp_prefix = "model."
    tie = {"lm_head.weight": "model.language_model.embed_tokens.weight"}
    # regex -> replacement, first match wins: brings the key layout of older transformers releases (sub-models under
    # ``language_model.model`` / ``vision_tower``) to the one the current classes (and the trainer) use
    key_map: Dict[str, str] = {}

    @classmethod
    def _rename(cls, key: str) -> str:
        import re
        for pat, rep in cls.key_map.items():
            new, n = re.subn(pat, rep, key)
            if n:
                return new
        return key

    @classmethod
    def hf_to_dcp(cls, cfg):
        import torch.distributed.checkpoint as dcp
        sd = hfio.load_state_dict(cfg["hf_dir"])
        if cfg.get("tie_weight"):
            for dst, src in cls.tie.items():
                if src in sd:
                    sd[dst] = sd[src]
        out = {}
        for k, v in sd.items():
            if any(n in k for n in cls.fused_linear_names) and v.dim() == 3:
                v = v.reshape(-1, v.shape[-1])
            out[cls.dcp_prefix + cls._rename(k)] = v
        dcp.save({"model": out}, checkpoint_id=os.path.join(cfg["dcp_dir"], "release"), no_dist=True)
        with open(os.path.join(cfg["dcp_dir"], "latest_checkpointed_iteration.txt"), "w") as f:
            f.write("release")

    @classmethod
    def dcp_to_hf(cls, cfg):
        from torch.distributed.checkpoint.format_utils import dcp_to_torch_save
        src = cfg.get("load_dir") or cfg["dcp_dir"]
        tr = os.path.join(src, "latest_checkpointed_iteration.txt")
        if os.path.exists(tr):
            tag = open(tr).read().strip()
            src = os.path.join(src, tag if tag == "release" else f"iter_{int(tag):07d}")
        save_dir = cfg.get("save_dir") or cfg["save_hf_dir"]
        assets = cfg.get("model_assets_dir") or cfg.get("hf_dir")
        os.makedirs(save_dir, exist_ok=True)
        tmp = os.path.join(save_dir, "_dcp_tmp.pt")
        dcp_to_torch_save(src, tmp)
        sd = torch.load(tmp, map_location="cpu", weights_only=False)
        os.remove(tmp)
        sd = sd.get("model", sd)
        n_exp = 0
        if assets and os.path.exists(os.path.join(assets, "config.json")):
            with open(os.path.join(assets, "config.json")) as f:
                c = json.load(f)
            n_exp = int(c.get("text_config", c).get("num_experts") or 0)
        out = {}
        for k, v in sd.items():
            if not isinstance(v, torch.Tensor):
                continue
            if n_exp and any(n in k for n in cls.fused_linear_names) and v.dim() == 2:
                v = v.reshape(n_exp, -1, v.shape[-1])
            if cfg.get("to_bf16"):
                v = v.to(torch.bfloat16)
            out[k[len(cls.dcp_prefix):] if k.startswith(cls.dcp_prefix) else k] = v
        hfio.save_sharded(out, save_dir)
        if assets:
            for f in os.listdir(assets):
                if f.endswith((".json", ".txt", ".jinja")) and f != hfio.INDEX:
                    import shutil
                    shutil.copy(os.path.join(assets, f), os.path.join(save_dir, f))

    @classmethod
    def moe_expert(cls, cfg):
        """``--cfg.style merge|split``: per-expert ``...experts.{e}.{gate,up,down}_proj.weight`` tensors of a Hugging Face MoE
        checkpoint <-> the fused ``gate_up_proj [E, H, 2F]`` / ``down_proj [E, F, H]`` pair (checkpoint/vlm_model/converters/
        moe_expert.py:55-121)."""
        from .operators import ExpertStack, Merge
        sd = hfio.load_state_dict(cfg["hf_dir"])
        base = cfg.get("weight_path", "model.language_model.layers.{i}.mlp.experts")
        ops = [Merge([base + ".{e}.gate_proj.weight", base + ".{e}.up_proj.weight"], base + ".{e}.gate_up.weight"),
               ExpertStack(base + ".{e}.gate_up.weight", base + ".gate_up_proj"),
               ExpertStack(base + ".{e}.down_proj.weight", base + ".down_proj")]
        if cfg.get("style", "merge") == "merge":
            for op in ops:
                op.apply(sd)
        else:
            for op in reversed(ops):
                op.revert(sd)
        hfio.save_sharded(sd, cfg["save_dir"])


@register
class Qwen3VLConverter(_DcpHFConverter):
    pass


@register
class Qwen35Converter(_DcpHFConverter):
    tie = {"lm_head.weight": "model.language_model.embed_tokens.weight"}


_LLAVA_STYLE = {r"^language_model\.model": "model.language_model", r"^vision_tower": "model.vision_tower",
                r"^multi_modal_projector": "model.multi_modal_projector", r"^language_model\.lm_head": "lm_head"}


@register
class InternVLConverter(_DcpHFConverter):
    """InternVL3 / InternVL3.5 (checkpoint/vlm_model/converters/internvl.py): ``hf_to_dcp`` / ``dcp_to_hf`` with the
    sub-model prefixes of older exports renamed, ``moe_expert`` for the 30B-A3B and 241B-A28B checkpoints."""
    key_map = _LLAVA_STYLE


@register
class Mistral3Converter(_DcpHFConverter):
    """Mistral-Small-3 / Magistral (checkpoint/vlm_model/converters/mistral3.py:38-46: the same renames)."""
    key_map = _LLAVA_STYLE
    fused_linear_names = ("gate_up_proj", "down_proj")


@register
class GlmConverter(_DcpHFConverter):
    """GLM-4.1V / GLM-4.5V (checkpoint/vlm_model/converters/glm.py): keys already follow the current layout."""


@register
class GenericDcpConverter(_DcpHFConverter):
    """Any Hugging Face checkpoint <-> the trainer's DCP layout with unchanged parameter names (``model_id: hf_auto``
    and every model whose internal names are the checkpoint's; checkpoint/fsdp/generic_dcp_converter.py)."""
    fused_linear_names = ()


@register
class LoraConverter:
    """``merge_lora_to_base``: fold a PEFT adapter (``adapter_model.safetensors`` + ``adapter_config.json``) into the base
    Hugging Face checkpoint, ``W += (alpha / r) * B @ A`` per target module (checkpoint/common/
    merge_lora_safetensors_to_base.py, merge_base_lora_weight.py)."""

    @staticmethod
    def merge_lora_to_base(cfg):
        from safetensors.torch import load_file
        base = hfio.load_state_dict(cfg["base_dir"])
        lora_dir = cfg["lora_dir"]
        ad = load_file(os.path.join(lora_dir, "adapter_model.safetensors"))
        with open(os.path.join(lora_dir, "adapter_config.json")) as f:
            ac = json.load(f)
        scale = float(cfg.get("scale") or ac["lora_alpha"] / ac["r"])
        merged, pre = 0, "base_model.model."
        for k, a in ad.items():
            if not k.endswith(".lora_A.weight"):
                continue
            stem = k[:-len(".lora_A.weight")]
            b = ad[stem + ".lora_B.weight"]
            name = (stem[len(pre):] if stem.startswith(pre) else stem) + ".weight"
            if name not in base:
                raise KeyError(f"adapter target {name} is not in the base checkpoint")
            w = base[name]
            base[name] = (w.float() + scale * (b.float() @ a.float())).to(w.dtype)
            merged += 1
        if not merged:
            raise ValueError(f"no lora_A / lora_B pairs in {lora_dir}")
        hfio.save_sharded(base, cfg["save_dir"])
        for f in os.listdir(cfg["base_dir"]):
            if f.endswith((".json", ".txt", ".jinja")) and f != hfio.INDEX:
                import shutil
                shutil.copy(os.path.join(cfg["base_dir"], f), os.path.join(cfg["save_dir"], f))
        print(f"merged {merged} adapter pairs (scale {scale:g}) into {cfg['save_dir']}")


@register
class HunyuanVideoConverter:
    """``source_to_mm`` / ``mm_to_source``: the published HunyuanVideo transformer file <-> this framework's parameter names
    (``checkpoint/hf.py: hunyuanvideo_ops``; the reference's checkpoint/sora_model/hunyuanvideo_converter.py:202-210)."""

    @staticmethod
    def _cfg(cfg):
        from ..models.mmdit import MMDiTConfig
        return MMDiTConfig.hunyuan_video()

    @classmethod
    def source_to_mm(cls, cfg):
        src = cfg["source_path"]
        sd = hfio.load_state_dict(src) if os.path.isdir(src) else _load_single(src)
        hfio.save_sharded(hfio.to_internal(sd, hfio.hunyuanvideo_ops(cls._cfg(cfg))), cfg["target_path"])

    @classmethod
    def mm_to_source(cls, cfg):
        sd = hfio.load_state_dict(cfg["source_path"])
        hfio.save_sharded(hfio.to_hf(sd, hfio.hunyuanvideo_ops(cls._cfg(cfg)), modern_prefix=False), cfg["target_path"])


def _load_single(path: str) -> Dict[str, torch.Tensor]:
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file
        return load_file(path)
    sd = torch.load(path, map_location="cpu", weights_only=True)
    return sd.get("module", sd)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 2 or argv[0] in ("-h", "--help"):
        print(__doc__)
        print("converters:", ", ".join(sorted(CONVERTERS)))
        return 0 if argv and argv[0] in ("-h", "--help") else 2
    conv, cmd = argv[0], argv[1]
    if conv not in CONVERTERS:
        raise SystemExit(f"unknown converter {conv}; known: {sorted(CONVERTERS)}")
    fn = getattr(CONVERTERS[conv], cmd, None)
    if fn is None:
        raise SystemExit(f"{conv} has no command {cmd}")
    fn(parse_cfg(argv[2:]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
