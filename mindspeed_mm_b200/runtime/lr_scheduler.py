"""Learning-rate schedules as pure functions of the step.

Same three shapes as mindspeed_mm/fsdp/optimizer/lr_scheduler.py:115-210: linear warm-up from
``lr_start`` to ``lr``, then constant / linear decay to ``lr_min`` / cosine decay over
``train_iters * lr_decay_ratio`` steps and ``lr_min`` afterwards.  The engine applies updates
inside backward, so the schedule is queried *before* a step rather than stepped after it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass
class LRSchedule:
    lr: float
    train_iters: int
    lr_decay_style: str = "cosine"
    lr_warmup_steps: int = 0
    lr_warmup_ratio: float = 0.0
    lr_min: float = 1e-7
    lr_start: float = 0.0
    lr_decay_ratio: float = 1.0
    num_cycles: float = 0.5

    def __post_init__(self):
        if self.lr_warmup_steps == 0 and self.lr_warmup_ratio > 0:
            self.lr_warmup_steps = int(self.train_iters * self.lr_warmup_ratio)
        if self.lr_decay_style not in ("constant", "linear", "cosine"):
            raise ValueError(f"Unknown learning rate decay style: {self.lr_decay_style}.")

    def __call__(self, step: int) -> float:
        lr, w = self.lr, self.lr_warmup_steps
        if lr == 0:
            return 0.0
        if step < w:
            return self.lr_start + (lr - self.lr_start) * step / max(1, w)
        if self.lr_decay_style == "constant":
            return lr
        if self.lr_decay_style == "linear":
            return lr * max(self.lr_min / lr, (self.train_iters - step) / max(1, self.train_iters - w))
        decay_steps = int(self.train_iters * self.lr_decay_ratio)
        if step > decay_steps:
            return self.lr_min
        progress = (step - w) / max(1, decay_steps - w)
        factor = 0.5 * (1.0 + math.cos(math.pi * self.num_cycles * 2.0 * progress))
        ratio = self.lr_min / lr
        return lr * max(0.0, factor * (1 - ratio) + ratio)

    def state_dict(self):
        return dict(self.__dict__)

    def load_state_dict(self, sd):
        self.__dict__.update(sd)
