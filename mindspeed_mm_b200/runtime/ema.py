"""Exponential moving average of the sharded fp32 master weights (mindspeed_mm/utils/ema.py).

The EMA lives next to each rank's master slice, so it costs 4 bytes per owned parameter and needs no
communication; ``swap`` exchanges EMA and live weights (evaluation / export), ``swap`` again restores them.
"""
from __future__ import annotations

import torch


class ShardedEMA:
    def __init__(self, engine, decay: float = 0.9999, update_after: int = 0):
        self.engine, self.decay, self.update_after, self.steps = engine, decay, update_after, 0
        self.shadow = {id(g): g.master.clone() for u in engine.units for g in u.groups if g.trainable}

    @torch.no_grad()
    def update(self):
        self.steps += 1
        d = 0.0 if self.steps <= self.update_after else min(self.decay, (1 + self.steps) / (10 + self.steps))
        for u in self.engine.units:
            for g in u.groups:
                if g.trainable:
                    self.shadow[id(g)].mul_(d).add_(g.master, alpha=1 - d)

    @torch.no_grad()
    def swap(self):
        for u in self.engine.units:
            for g in u.groups:
                if g.trainable:
                    s = self.shadow[id(g)]
                    tmp = g.master.clone()
                    g.master.copy_(s)
                    g.shard16.copy_(s)
                    s.copy_(tmp)

    def state_dict(self):
        return {"steps": self.steps, "shadow": [self.shadow[id(g)] for u in self.engine.units for g in u.groups if g.trainable]}

    def load_state_dict(self, sd):
        self.steps = sd["steps"]
        it = iter(sd["shadow"])
        for u in self.engine.units:
            for g in u.groups:
                if g.trainable:
                    self.shadow[id(g)].copy_(next(it))
