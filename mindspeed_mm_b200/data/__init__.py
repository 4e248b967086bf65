"""Datasets, samplers, collators and loaders.

``build_dataloader(args, model, parallel_state, device)`` resolves ``data.dataset_param.dataset_type`` in the
dataset registry, builds the sampler named by ``dataloader_param.sampler_type``, the collator (packing for
VLMs) and returns ``(train_iterator, val_iterator_factory)``; reference: mindspeed_mm/data/__init__.py:30-97 and
mindspeed_mm/fsdp/data/__init__.py:9-34.
"""
from __future__ import annotations

from typing import Callable, Iterator, Optional, Tuple

import torch
from torch.utils.data import DataLoader

from ..models.registry import data_register
from . import synthetic  # noqa: F401  (registers the synthetic datasets)
from . import anyres  # noqa: F401  (registers the tiled conversation dataset)
from . import multimodal  # noqa: F401  (registers huggingface / multimodal / feature / t2v / i2v)
from . import internvl  # noqa: F401  (registers the dynamic-tile conversation dataset)


class _StatefulIter:
    """Infinite iterator over a DataLoader that exposes the sampler's resumable state."""

    def __init__(self, loader: DataLoader, sampler):
        self.loader, self.sampler = loader, sampler
        self._it = iter(loader)

    def __iter__(self):
        return self

    def __next__(self):
        try:
            return next(self._it)
        except StopIteration:
            self._it = iter(self.loader)
            return next(self._it)

    def state_dict(self):
        return self.sampler.state_dict() if hasattr(self.sampler, "state_dict") else None

    def load_state_dict(self, s):
        if s is not None and hasattr(self.sampler, "load_state_dict"):
            self.sampler.load_state_dict(s)
            self._it = iter(self.loader)


def _vision_of(cfg):
    """The vision tower's config: ``vision`` on the per-family configs, ``vit`` on the composable one when its tower is the
    plain ViT."""
    v = getattr(cfg, "vision", None)
    return v if v is not None else getattr(cfg, "vit", None)


def build_dataset(dataset_param, model=None):
    kind = dataset_param.dataset_type
    cls = data_register.get(kind)
    basic = dict(dataset_param.basic_parameters or {})
    if kind == "synthetic_vlm":
        from .synthetic import SyntheticVLMSpec
        cfg = getattr(model, "config", None)
        if cfg is not None:
            basic.setdefault("vocab_size", cfg.text.vocab_size)
            basic.setdefault("image_token_id", cfg.image_token_id)
            basic.setdefault("vision_start_token_id", cfg.vision_start_token_id)
            v = _vision_of(cfg)
            if v is not None:
                basic.setdefault("patch", v.patch_size)
                basic.setdefault("merge", getattr(v, "spatial_merge_size", getattr(v, "merge", 2)) or 2)
                basic.setdefault("temporal_patch", getattr(v, "temporal_patch_size", 2))
            else:                           # no vision tower (speech / text decoders): text-only samples
                basic["images_per_sample"] = 0
        return cls(SyntheticVLMSpec(**basic))
    if kind == "synthetic_asr":
        from .synthetic import SyntheticASRSpec
        cfg = getattr(model, "config", None)
        if cfg is not None and getattr(cfg, "audio", None) is not None:
            basic.setdefault("vocab_size", cfg.text.vocab_size)
            basic.setdefault("audio_token_id", cfg.audio_token_id)
            basic.setdefault("n_mels", cfg.audio.num_mel_bins)
            basic.setdefault("n_window", cfg.audio_window)
        return cls(SyntheticASRSpec(**basic))
    if kind == "synthetic_av_latents":
        from .synthetic import SyntheticAVLatentSpec
        return cls(SyntheticAVLatentSpec(**basic))
    if kind == "synthetic_speech":
        from .synthetic import SyntheticSpeechSpec
        return cls(SyntheticSpeechSpec(**basic))
    if kind == "synthetic_video_latents":
        from .synthetic import SyntheticVideoLatentSpec
        return cls(SyntheticVideoLatentSpec(**basic))
    return cls(dataset_param, model=model)


def build_collator(args, model, pin: bool):
    cp = args.data.dataloader_param.collate_param
    name = (cp.collator_id or cp.model_name or "").lower()
    cfg = getattr(model, "config", None)
    if hasattr(model, "collate"):                 # models with their own sequence layout (speech LMs) pack their samples
        return model.collate
    if args.data.dataset_param.dataset_type == "deepseekvl2" or "deepseek" in name:
        from .anyres import TiledPackCollator
        vit = cfg.vit
        return TiledPackCollator(vit.patch_size, vit.merge, vit.temporal_patch_size)
    if args.data.dataset_param.dataset_type == "synthetic_asr":
        from .synthetic import ASRPackCollator
        return ASRPackCollator()
    if args.data.dataset_param.dataset_type == "internvl" or "internvl" in name:
        from .internvl import TilePackCollator
        return TilePackCollator.for_config(cfg, pin=pin)
    if "qwen2" in name or "vl" in name or args.data.dataset_param.dataset_type == "synthetic_vlm":
        from .collate import PackedVLMCollator
        return PackedVLMCollator.for_config(cfg, pin=pin)
    return lambda samples: {k: torch.stack([s[k] for s in samples]) for k in samples[0]}


def build_dataloader(args, model, ps, device) -> Tuple[Iterator, Optional[Callable[[], Iterator]]]:
    from .samplers import SAMPLERS
    dl = args.data.dataloader_param
    ds = build_dataset(args.data.dataset_param, model)
    n = len(ds)
    sampler_cls = SAMPLERS.get(dl.sampler_type, SAMPLERS["BaseRandomBatchSampler"])
    sampler = sampler_cls(n, args.training.micro_batch_size, ps.get_dp_rank(), ps.get_dp_world_size(),
                          seed=args.training.seed, shuffle=bool(dl.shuffle), drop_last=dl.drop_last)
    pin = dl.pin_memory and torch.cuda.is_available()
    loader = DataLoader(ds, batch_sampler=sampler, collate_fn=build_collator(args, model, pin), num_workers=dl.num_workers,
                        persistent_workers=dl.num_workers > 0)
    it: Iterator = _StatefulIter(loader, sampler)
    if dl.enable_preload:
        from .preloader import Preloader
        inner = it
        pre = Preloader(inner, device)
        pre.state_dict, pre.load_state_dict = inner.state_dict, inner.load_state_dict
        it = pre
    val_fn = None
    if args.data.val_dataset_param is not None:
        vds = build_dataset(args.data.val_dataset_param, model)
        coll = build_collator(args, model, False)
        mbs = args.training.val_micro_batch_size or args.training.micro_batch_size

        def val_fn():
            for s in range(ps.get_dp_rank() * mbs, len(vds) - mbs + 1, mbs * ps.get_dp_world_size()):
                yield coll([vds[i] for i in range(s, s + mbs)])
    return it, val_fn
