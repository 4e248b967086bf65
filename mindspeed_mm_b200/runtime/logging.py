"""Console log lines.

The iteration line keeps the exact field names of the reference (`elapsed time per iteration (ms)`,
`tokens per sample`, ...) because its launch scripts and CI scrape them with awk/regex
(examples/qwen2.5vl/finetune_qwen2_5_vl_7b.sh:115-123, tests/st/test_tools/acquire_json.py:29-62);
format: mindspeed_mm/fsdp/train/train_engine.py:343-359 and mindspeed_mm/training.py:1022-1071.
"""
from __future__ import annotations

import logging
import os
import sys
from datetime import datetime
from typing import Dict, Optional

import torch

_LOGGER = None


class _StdoutHandler(logging.StreamHandler):
    """Writes to whatever ``sys.stdout`` is at the time of the record (redirections made after the logger was created,
    e.g. by a launcher or a test harness, are honoured)."""

    def __init__(self):
        logging.Handler.__init__(self)

    @property
    def stream(self):
        return sys.stdout

    @stream.setter
    def stream(self, _value):
        pass


def get_logger(name: str = "mm_b200") -> logging.Logger:
    global _LOGGER
    if _LOGGER is None:
        lg = logging.getLogger(name)
        if not lg.handlers:
            h = _StdoutHandler()
            h.setFormatter(logging.Formatter("%(message)s"))
            lg.addHandler(h)
        lg.setLevel(os.environ.get("MM_B200_LOGLEVEL", "INFO"))
        lg.propagate = False
        _LOGGER = lg
    return _LOGGER


def is_rank0() -> bool:
    return int(os.environ.get("RANK", "0")) == 0


def print_rank0(msg: str) -> None:
    if is_rank0():
        get_logger().info(msg)


def format_training_log(iteration: int, train_iters: int, consumed_samples: int, elapsed_s: float, lr: float,
                        global_batch_size: int, loss_dict: Dict[str, float], grad_norm: Optional[float] = None,
                        tokens_per_sample: Optional[float] = None, loss_scale: Optional[float] = None,
                        skipped: int = 0, nan_iters: int = 0) -> str:
    s = f" [{datetime.now().strftime('%Y-%m-%d %H:%M:%S')}]"
    s += " iteration {:8d}/{:8d} |".format(iteration, train_iters)
    s += " consumed samples: {:12d} |".format(consumed_samples)
    s += " elapsed time per iteration (ms): {:.1f} |".format(elapsed_s * 1000.0)
    s += " learning rate: {:.6E} |".format(lr)
    s += " global batch size: {:5d} |".format(global_batch_size)
    if tokens_per_sample is not None:
        s += " tokens per sample: {:.1f} |".format(tokens_per_sample)
    for name, value in loss_dict.items():
        s += f" {name}: {value:.6E} |"
    if loss_scale is not None:
        s += " loss scale: {:.1f} |".format(loss_scale)
    if grad_norm is not None:
        s += " grad norm: {:.3f} |".format(grad_norm)
    if skipped or nan_iters:
        s += " number of skipped iterations: {:3d} |".format(skipped)
        s += " number of nan iterations: {:3d} |".format(nan_iters)
    return s


def format_memory_report(rank: int, iteration: int) -> str:
    mb = 1024.0 * 1024.0
    if not torch.cuda.is_available():
        return f"[Rank {rank}] (after {iteration} iterations) memory (MB) | allocated: 0 | max allocated: 0 | reserved: 0 | max reserved: 0"
    return ("[Rank {}] (after {} iterations) memory (MB) | allocated: {} | max allocated: {} | reserved: {} | "
            "max reserved: {}").format(rank, iteration, torch.cuda.memory_allocated() / mb,
                                        torch.cuda.max_memory_allocated() / mb, torch.cuda.memory_reserved() / mb,
                                        torch.cuda.max_memory_reserved() / mb)


class ScalarLog:
    """Per-iteration scalars for dashboards, written by rank 0: a TensorBoard event file (``tensorboard_dir``), a Weights &
    Biases run (``wandb_project``; when the package is missing or cannot start a run, e.g. no login or no network, the
    same records go to ``wandb-offline.jsonl`` in ``wandb_dir``), or both.  Every scalar is written against the iteration and, as ``"<name> vs samples"``, against the
    consumed samples, the pairing the reference's training log uses (mindspeed_mm/training.py:934-1007)."""

    def __init__(self, tensorboard_dir: Optional[str] = None, wandb_project: Optional[str] = None,
                 wandb_dir: Optional[str] = None, wandb_name: Optional[str] = None, interval: int = 1):
        self.interval = max(1, int(interval))
        self.tb = self.wb = self.jsonl = None
        if not is_rank0():
            return
        if tensorboard_dir:
            from torch.utils.tensorboard import SummaryWriter
            os.makedirs(tensorboard_dir, exist_ok=True)
            self.tb = SummaryWriter(log_dir=tensorboard_dir)
        if wandb_project:
            try:
                import wandb
                self.wb = wandb.init(project=wandb_project, name=wandb_name, dir=wandb_dir)
            except Exception:  # noqa: BLE001  (package missing, no login, no network: keep the records locally)
                d = wandb_dir or tensorboard_dir or "."
                os.makedirs(d, exist_ok=True)
                self.jsonl = open(os.path.join(d, "wandb-offline.jsonl"), "a")

    @property
    def active(self) -> bool:
        return self.tb is not None or self.wb is not None or self.jsonl is not None

    def log(self, iteration: int, consumed_samples: int, scalars: Dict[str, float]) -> None:
        if not self.active or iteration % self.interval:
            return
        scalars = {k: float(v) for k, v in scalars.items() if v is not None}
        if self.tb is not None:
            for k, v in scalars.items():
                self.tb.add_scalar(k, v, iteration)
                self.tb.add_scalar(k + " vs samples", v, consumed_samples)
        if self.wb is not None:
            self.wb.log(dict(scalars, **{"samples vs steps": consumed_samples}), step=iteration)
        if self.jsonl is not None:
            import json
            self.jsonl.write(json.dumps(dict(scalars, iteration=iteration, samples=consumed_samples)) + "\n")
            self.jsonl.flush()

    def close(self) -> None:
        if self.tb is not None:
            self.tb.close()
        if self.wb is not None:
            self.wb.finish()
        if self.jsonl is not None:
            self.jsonl.close()

