"""Any Hugging Face ``PreTrainedModel`` under the ZeRO-3 engine.

The native models of this package call their sharding units through ``run(module, ...)``.  A transformers class calls
its sub-modules itself, so the adapter re-routes instead: every module that becomes a unit (the classes the model names
in ``_no_split_modules``, and for every parameter outside those the module that holds it: embeddings, norms, the output
head) gets an instance-level ``forward`` that hands the call to ``engine.run``; the engine then runs the class-level
forward with the parameters gathered (and recomputes it in the backward).  Nothing inside transformers is edited.

Reference: mindspeed_mm/fsdp/models/modelhub.py:60-70 (stock transformers class built on the meta device),
fsdp/distributed/fully_shard_parallel.py:42-109 (``fully_shard`` applied to the modules a recipe lists, then the root),
mindspeed_mm/models/transformers/*.py (per-family registration of those classes).

    model = AutoModelForCausalLM.from_config(cfg)          # or from_pretrained
    adapter = HFModelAdapter(model)
    engine = FSDPEngine(adapter.fsdp_units(), ...)
    adapter.attach(engine)
    loss_sum, n = adapter(batch)                            # packed batch of the VLM collators, or input_ids [B, S]
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class HFModelAdapter(nn.Module):
    """Wraps ``model`` (a ``PreTrainedModel``) with the training interface of the native models: ``fsdp_units()``,
    ``forward(batch, run=None) -> (loss_sum, n_valid)`` or logits.

    Units: every top-level instance of a class in ``unit_classes`` (default: the model's ``_no_split_modules``); then, for
    each parameter not covered yet, the module that holds it directly (embeddings, norms, projections, the output head).
    An output head tied to the input embedding is untied (a copy), because the two live in different units."""

    def __init__(self, model: nn.Module, unit_classes: Optional[Sequence[str]] = None, ignore_index: int = -100,
                 use_plugin_attention: bool = False):
        super().__init__()
        self.model = model
        self.config = model.config
        self.ignore_index = ignore_index
        self._untie(model)
        names = set(unit_classes or getattr(model, "_no_split_modules", None) or ())
        units: Dict[str, nn.Module] = {}
        for name, mod in model.named_modules():
            if name and type(mod).__name__ in names and not any(name.startswith(t + ".") for t in units):
                units[name] = mod
        owned = {id(p) for m in units.values() for p in m.parameters()}
        for name, mod in model.named_modules():
            mine = [p for p in mod.parameters(recurse=False) if id(p) not in owned]
            if not mine:
                continue
            if not name or any(u.startswith(name + ".") for u in units):
                raise ValueError(f"parameters held directly by '{name or type(model).__name__}' cannot form a unit: the "
                                 f"module also contains other units; list its class in unit_classes instead")
            units[name] = mod
            owned.update(id(p) for p in mod.parameters())
        self._unit_modules: List[Tuple[str, nn.Module]] = [(n, m) for n, m in model.named_modules() if n in units]
        if use_plugin_attention:
            from .hf_kernels import use_plugin_attention as _use
            _use(model, packed_towers=use_plugin_attention == "packed_towers")
        self._engine = None
        text_cfg = model.config.get_text_config() if hasattr(model.config, "get_text_config") else model.config
        rope = getattr(text_cfg, "rope_parameters", None) or getattr(text_cfg, "rope_scaling", None) or {}
        self._mrope = isinstance(rope, dict) and "mrope_section" in rope
        impl = getattr(model.config, "_attn_implementation", None) or ""
        self._varlen_kwargs = impl == "mm_b200" or "flash" in impl
        import inspect
        self._forward_params = [n for n, p in inspect.signature(model.forward).parameters.items()
                                if p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)]

    @staticmethod
    def _untie(model) -> None:
        head = model.get_output_embeddings() if hasattr(model, "get_output_embeddings") else None
        emb = model.get_input_embeddings() if hasattr(model, "get_input_embeddings") else None
        if head is not None and emb is not None and getattr(head, "weight", None) is getattr(emb, "weight", 0):
            head.weight = nn.Parameter(emb.weight.detach().clone(), requires_grad=emb.weight.requires_grad)
            for c in (model.config, getattr(model.config, "text_config", None)):
                if c is not None and hasattr(c, "tie_word_embeddings"):
                    c.tie_word_embeddings = False
            names = {id(m): n for n, m in model.named_modules()}
            # a checkpoint of the tied model stores the matrix once: the load fills the head from the embedding
            model._untied_head = (names[id(emb)] + ".weight", names[id(head)] + ".weight")

    # -- sharding plan ---------------------------------------------------------------------------------------------
    def fsdp_units(self) -> List[Tuple[str, nn.Module]]:
        # the engine swaps the parameters for views of its flat buffers: keep the loaded values until ``attach``
        self._initial = {n: p.data for n, p in self.model.named_parameters() if not p.is_meta}
        return [("model." + n, m) for n, m in self._unit_modules]

    def attach(self, engine, materialize: bool = True) -> None:
        """Route the unit modules' calls through ``engine.run``; the engine itself calls the class-level forward.
        ``materialize``: allocate the engine's shards and fill them with the values the model held when the units were
        listed (a model built on the meta device is filled by a checkpoint load instead)."""
        self._engine = engine
        self._materialize_buffers(engine.device)
        initial, self._initial = getattr(self, "_initial", {}), {}
        if materialize:
            def init(unit_name: str, mod: nn.Module):
                base = unit_name[len("model."):]
                for k, p in mod.named_parameters():
                    src = initial.get(f"{base}.{k}")
                    if src is not None:
                        p.data.copy_(src)
            engine.materialize(init)
        for _, mod in self._unit_modules:
            u = engine._by_module.get(id(mod))
            if u is None:
                continue
            u.call = (lambda m: lambda *a, **k: type(m).forward(m, *a, **k))(mod)
            mod.forward = (lambda m: lambda *a, **k: engine.run(m, *a, **k))(mod)

    @torch.no_grad()
    def _materialize_buffers(self, device) -> None:
        """A model built on the meta device has its buffers there too (rotary inverse frequencies).  The engine only
        owns parameters, so buffers are allocated here and filled by the model's own ``_init_weights``, which is where
        transformers recomputes them after a meta-device build."""
        for name, mod in self.model.named_modules():
            meta = [k for k, b in mod._buffers.items() if b is not None and b.is_meta]
            if not meta:
                continue
            if any(True for _ in mod.parameters(recurse=False)) or not hasattr(self.model, "_init_weights"):
                raise NotImplementedError(f"'{name}' ({type(mod).__name__}) holds buffers on the meta device next to "
                                          f"parameters; build the model on a real device instead")
            for k in meta:
                mod._buffers[k] = torch.empty_like(mod._buffers[k], device=device)
            self.model._init_weights(mod)

    def detach(self) -> None:
        for _, mod in self._unit_modules:
            mod.__dict__.pop("forward", None)
        self._engine = None

    # -- forward ---------------------------------------------------------------------------------------------------
    def forward(self, batch: dict, run=None):
        ids = batch["input_ids"]
        packed = ids.dim() == 1
        kw: Dict[str, object] = {}
        if packed:                          # one packed row: sequences are told apart by their positions
            kw["input_ids"] = ids[None]
            pos = batch.get("position_ids")
            cu = batch.get("cu_seqlens")
            if pos is None and cu is not None and cu.numel() > 2:        # several sequences: positions restart in each
                cu = cu.long()
                tok = torch.arange(ids.numel(), device=ids.device)
                seq = torch.bucketize(tok, cu[1:], right=True).clamp(max=cu.numel() - 2)
                pos = tok - cu[seq]
            if cu is not None and cu.numel() > 2 and self._varlen_kwargs:
                # attention implementations that take packed rows by their boundaries (flash-attention style, "mm_b200")
                # get them explicitly; mask-based ones derive the block-diagonal mask from the positions
                cu32 = cu.to(device=ids.device, dtype=torch.int32)
                longest = int(batch.get("max_seqlen") or int((cu32[1:] - cu32[:-1]).max()))
                kw.update(cu_seq_lens_q=cu32, cu_seq_lens_k=cu32, max_length_q=longest, max_length_k=longest)
            if pos is not None:             # [T], or [3, T] multimodal positions of the VLM collators
                if pos.dim() == 2 and not self._mrope:
                    pos = pos[0]            # a decoder with 1-D rotary positions: the temporal row is the token position
                kw["position_ids"] = pos[None] if pos.dim() == 1 else pos[:, None]
        else:
            kw["input_ids"] = ids
            if batch.get("attention_mask") is not None:
                kw["attention_mask"] = batch["attention_mask"]
        # every other batch entry the architecture's forward names goes through (pixel_values, image_grid_thw, image_sizes,
        # input_features, ...); empty media tensors are left out
        for k in self._forward_params:
            if k in kw or k in ("labels", "input_ids", "attention_mask", "position_ids", "use_cache", "past_key_values"):
                continue
            val = batch.get(k)
            if val is not None and (not torch.is_tensor(val) or val.numel() > 0):
                kw[k] = val
        logits = self.model(**kw, use_cache=False).logits
        labels = batch.get("labels")
        if labels is None:
            return logits[0] if packed else logits
        flat = logits.reshape(-1, logits.shape[-1]).float()
        lab = labels.reshape(-1)                    # already shifted by the collators (label t = token t + 1)
        loss_sum = F.cross_entropy(flat, lab, ignore_index=self.ignore_index, reduction="sum")
        return loss_sum, (lab != self.ignore_index).sum()
