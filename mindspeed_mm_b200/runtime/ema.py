"""Exponential moving averages of the trained weights (mindspeed_mm/utils/ema.py; used by the reference's autoencoder
training, mindspeed_mm/models/ae/training/training.py:143-146,207-208,244).

* ``ShardedEMA`` -- for the sharding engine: the average lives next to each rank's fp32 master slice (4 bytes per owned
  parameter, on the device or on the host wherever the master is), needs no communication, is part of the per-rank
  checkpoint state; ``swap`` exchanges average and live weights (evaluation / export) and ``swap`` again restores them.
* ``ModuleEMA``  -- for a plain ``nn.Module`` trained by a torch optimizer (the autoencoder trainer):
  ``shadow = decay * shadow + (1 - decay) * param`` after every step, ``apply_shadow`` / ``restore`` around evaluation.
"""
from __future__ import annotations

import torch


def _groups(engine):
    engines = getattr(engine, "engines", None) or (engine,)
    return [g for e in engines for u in e.units for g in u.groups if g.trainable]


class ShardedEMA:
    def __init__(self, engine, decay: float = 0.9999, update_after: int = 0, warmup: bool = True):
        """``warmup``: the effective decay ramps as ``(1 + n) / (10 + n)`` until it reaches ``decay``."""
        self.engine, self.decay, self.update_after, self.warmup, self.steps = engine, decay, update_after, warmup, 0
        self.shadow = [g.master.clone() for g in _groups(engine)]

    @torch.no_grad()
    def update(self):
        self.steps += 1
        if self.steps <= self.update_after:
            d = 0.0
        else:
            d = min(self.decay, (1 + self.steps) / (10 + self.steps)) if self.warmup else self.decay
        for s, g in zip(self.shadow, _groups(self.engine)):
            s.mul_(d).add_(g.master, alpha=1 - d)

    @torch.no_grad()
    def swap(self):
        for s, g in zip(self.shadow, _groups(self.engine)):
            tmp = g.master.clone()
            g.master.copy_(s)
            g.shard16.copy_(s)
            s.copy_(tmp)

    def state_dict(self):
        return {"steps": self.steps, "shadow": [s.cpu() for s in self.shadow]}

    def load_state_dict(self, sd):
        self.steps = sd["steps"]
        for s, t in zip(self.shadow, sd["shadow"]):
            s.copy_(t)


class ModuleEMA:
    def __init__(self, module: torch.nn.Module, decay: float = 0.999):
        self.module, self.decay = module, decay
        self.shadow = {n: p.detach().clone() for n, p in module.named_parameters() if p.requires_grad}
        self.backup = {}

    @torch.no_grad()
    def update(self):
        for n, p in self.module.named_parameters():
            if n in self.shadow:
                self.shadow[n].mul_(self.decay).add_(p.detach(), alpha=1.0 - self.decay)

    @torch.no_grad()
    def apply_shadow(self):
        for n, p in self.module.named_parameters():
            if n in self.shadow:
                self.backup[n] = p.detach().clone()
                p.copy_(self.shadow[n])

    @torch.no_grad()
    def restore(self):
        for n, p in self.module.named_parameters():
            if n in self.backup:
                p.copy_(self.backup[n])
        self.backup = {}

    def state_dict(self):
        return dict(self.shadow)

    def load_state_dict(self, sd):
        for n, t in sd.items():
            self.shadow[n].copy_(t)
