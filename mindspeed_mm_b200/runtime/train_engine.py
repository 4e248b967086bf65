"""Training loop shared by every backend.

One loop (the reference has two: mindspeed_mm/training.py:346-708 for Megatron and
mindspeed_mm/fsdp/train/train_engine.py:131-319 for native FSDP): per iteration
``profilers.step -> [micro-batches: H2D, forward, loss, backward] -> finish (clip/update) ->
log -> validate -> save -> exit conditions``.  The optimizer lives inside the sharding engine,
because updates are applied as each unit's gradients are reduced.

Timing: ``elapsed time per iteration`` is wall time between iteration boundaries with a device
synchronise on each side (what the reference prints); benchmarks use CUDA events instead.
"""
from __future__ import annotations

import math
import os
import signal
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

from ..data.collate import to_device
from ..parallel.fsdp import FSDPEngine
from .logging import format_memory_report, format_training_log, print_rank0
from .lr_scheduler import LRSchedule


@dataclass
class TrainConfig:
    train_iters: int = 10
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    global_batch_size: Optional[int] = None
    log_interval: int = 1
    save_interval: int = 0
    val_interval: int = 0
    val_iters: int = 0
    exit_interval: int = 0
    exit_duration_in_mins: float = 0.0
    log_tps: bool = True
    report_memory_at: int = 1
    check_for_nan: bool = True


class NativeKernelTimeout(RuntimeError):
    """A native kernel gave up a bounded wait (on a peer flag, an mbarrier, the arena barrier) during the step that
    just ended: its outputs are incomplete, so the run stops instead of training on them.  ``exit_code`` is the code
    the host watchdog uses for a stalled step."""
    exit_code = 3


class TrainEngine:
    def __init__(self, model, engine: FSDPEngine, loss_fn: Callable, schedule: LRSchedule, cfg: TrainConfig,
                 data_iter: Optional[Iterable] = None, val_iter_fn: Optional[Callable[[], Iterable]] = None,
                 checkpointer=None, profiler=None, memory_profiler=None, watchdog=None, dp_group=None,
                 dp_world: int = 1, device="cpu", status_word: Optional[torch.Tensor] = None, ema=None,
                 scalar_log=None):
        self.model, self.engine, self.loss_fn, self.schedule, self.cfg = model, engine, loss_fn, schedule, cfg
        self.scalar_log = scalar_log      # runtime.logging.ScalarLog (TensorBoard / W&B), rank 0 writes
        self._aux = []                    # MoE load-balancing terms of the current step's micro-batches
        self._mtp = []                    # multi-token-prediction losses [depths] of the current step's micro-batches
        self.ema = ema            # runtime.ema.ShardedEMA: updated after every optimizer step, saved with the per-rank state
        self.data_iter, self.val_iter_fn = data_iter, val_iter_fn
        self.checkpointer, self.profiler, self.memory_profiler, self.watchdog = \
            checkpointer, profiler, memory_profiler, watchdog
        self.dp_group, self.dp_world = dp_group, dp_world
        self.device = torch.device(device)
        self.iteration = 0
        self.consumed_train_samples = 0
        self.nan_iters = 0
        self.skipped_iters = 0
        if cfg.global_batch_size is None:
            cfg.global_batch_size = cfg.micro_batch_size * cfg.gradient_accumulation_steps * dp_world
        self._sigterm = False
        self._t_start = time.time()
        self.history: List[Dict[str, float]] = []
        # int32[1] that kernels write when a bounded wait expires (0 = fine); read once per iteration in train()
        self.status_word = status_word
        if status_word is None and self.device.type == "cuda":
            from .. import ops
            if ops.get_tier() == "native":
                from ..ops import native
                self.status_word = native.status_word(self.device)

    # ---------------------------------------------------------------------------------- one step
    def forward_backward(self, batch: dict) -> Dict[str, torch.Tensor]:
        """One micro-batch on device tensors.  Returns detached scalars for logging."""
        out = self.model(batch, run=self.engine.run)
        if isinstance(out, tuple):
            loss_sum, n_valid = out[0], out[1]
            loss = self.loss_fn(loss_sum, n_valid)
        else:
            loss, n_valid = out, None
        loss.backward()
        # MoE router load-balancing term: its gradient is attached inside the MoE blocks (it flows in recomputed units
        # too); the model reports the value of this micro-batch for the log
        aux_fn = getattr(self.model, "aux_loss", None)
        aux = aux_fn() if callable(aux_fn) else None
        if aux is not None:
            self._aux.append(aux.detach())
        mtp = getattr(self.model, "last_mtp_losses", None)      # per-depth multi-token-prediction losses of this micro-batch
        if mtp:
            self._mtp.append(torch.stack(list(mtp)).float())
        self.engine.end_micro_step()
        return dict(loss=loss.detach(), n_valid=n_valid)

    def train_step(self, micro_batches: List[dict]) -> Dict[str, torch.Tensor]:
        """A full optimizer step over host (pinned) or device micro-batches."""
        self.engine.set_lr(self.schedule(self.iteration))
        losses, tokens = [], 0
        for mb in micro_batches:
            mb = to_device(mb, self.device) if self.device.type == "cuda" else mb
            r = self.forward_backward(mb)
            losses.append(r["loss"])
            tokens += int(mb.get("n_tokens", 0))
        grad_norm = self.engine.finish_step()
        if self.ema is not None:
            self.ema.update()
        loss = torch.stack(losses).mean()
        if self.dp_world > 1:
            dist.all_reduce(loss, op=dist.ReduceOp.AVG if loss.is_cuda else dist.ReduceOp.SUM, group=self.dp_group)
            if not loss.is_cuda:
                loss = loss / self.dp_world
        aux = None
        if self._aux:                       # tracker of the router's auxiliary loss: mean over micro-batches and data ranks
            aux = torch.stack(self._aux).float().mean()
            self._aux = []
            if self.dp_world > 1:
                dist.all_reduce(aux, group=self.dp_group)
                aux = aux / self.dp_world
        mtp = None
        if self._mtp:                       # tracker of the multi-token-prediction losses, one value per depth
            mtp = torch.stack(self._mtp).mean(0)
            self._mtp = []
            if self.dp_world > 1:
                dist.all_reduce(mtp, group=self.dp_group)
                mtp = mtp / self.dp_world
        self.iteration += 1
        self.consumed_train_samples += self.cfg.global_batch_size
        return dict(loss=loss, grad_norm=grad_norm, tokens=tokens, aux_loss=aux, mtp_losses=mtp)

    # ---------------------------------------------------------------------------------- loop
    def _sync(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def check_kernel_status(self) -> None:
        """Read the kernels' status word at an iteration boundary (the device is already synchronised there), take the
        maximum over all ranks so that every rank stops in the same iteration, and raise when it is not zero."""
        if self.status_word is None:
            return
        st = self.status_word
        if dist.is_initialized() and dist.get_world_size() > 1:
            st = st.clone()
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        code = int(st.item())
        if code != 0:
            self.status_word.zero_()
            raise NativeKernelTimeout(f"a native kernel gave up a bounded wait in iteration {self.iteration} "
                                      f"(status {code}); stopping before the next step")

    def train(self) -> List[Dict[str, float]]:
        cfg = self.cfg
        prev = signal.getsignal(signal.SIGTERM)
        try:
            signal.signal(signal.SIGTERM, lambda *_: setattr(self, "_sigterm", True))
        except ValueError:  # not the main thread
            prev = None
        it = iter(self.data_iter)
        if self.profiler:
            self.profiler.start()
        try:
            while self.iteration < cfg.train_iters:
                if self.memory_profiler:
                    self.memory_profiler.step(self.iteration)
                if self.watchdog:
                    self.watchdog.beat(self.iteration)
                self._sync()
                t0 = time.time()
                lr = self.schedule(self.iteration)
                mbs = [next(it) for _ in range(cfg.gradient_accumulation_steps)]
                r = self.train_step(mbs)
                self._sync()
                self.check_kernel_status()
                dt = time.time() - t0
                loss = float(r["loss"])
                if cfg.check_for_nan and not math.isfinite(loss):
                    self.nan_iters += 1
                rec = dict(iteration=self.iteration, loss=loss, time=dt, lr=lr,
                           grad_norm=None if r["grad_norm"] is None else float(r["grad_norm"]))
                if r.get("aux_loss") is not None:
                    rec["load_balancing_loss"] = float(r["aux_loss"])
                if r.get("mtp_losses") is not None:
                    for d, v in enumerate(r["mtp_losses"].tolist()):
                        rec[f"mtp_{d + 1} loss"] = v
                self.history.append(rec)
                if self.scalar_log is not None and self.scalar_log.active:
                    sc = {"lm loss": loss, "learning-rate": lr, "grad-norm": rec["grad_norm"], "batch-size": cfg.global_batch_size,
                          "iteration-time": dt, "load_balancing_loss": rec.get("load_balancing_loss")}
                    sc.update({k: v for k, v in rec.items() if k.startswith("mtp_")})
                    if self.device.type == "cuda":
                        ms = torch.cuda.memory_stats(self.device)
                        sc.update({"mem-reserved-bytes": ms["reserved_bytes.all.current"],
                                   "mem-allocated-bytes": ms["allocated_bytes.all.current"]})
                    self.scalar_log.log(self.iteration, self.consumed_train_samples, sc)
                if cfg.log_interval and self.iteration % cfg.log_interval == 0:
                    tps = r["tokens"] / max(1, cfg.micro_batch_size * cfg.gradient_accumulation_steps) \
                        if cfg.log_tps and r["tokens"] else None
                    print_rank0(format_training_log(self.iteration, cfg.train_iters, self.consumed_train_samples, dt,
                                                    lr, cfg.global_batch_size,
                                                    {"loss": loss, **{k: v for k, v in rec.items()
                                                                      if k == "load_balancing_loss" or k.startswith("mtp_")}},
                                                    rec["grad_norm"], tps,
                                                    skipped=self.skipped_iters, nan_iters=self.nan_iters))
                if self.iteration == cfg.report_memory_at:
                    if (dist.get_rank() if dist.is_initialized() else 0) == 0:
                        print(format_memory_report(0, self.iteration), flush=True)
                if cfg.val_interval and self.val_iter_fn and self.iteration % cfg.val_interval == 0:
                    self.validate()
                if self.profiler:
                    self.profiler.step()
                if self.checkpointer and cfg.save_interval and self.iteration % cfg.save_interval == 0:
                    self.save()
                if self._should_exit():
                    if self.checkpointer:
                        self.save()
                    break
        finally:
            if self.scalar_log is not None:
                self.scalar_log.close()
            if self.profiler:
                self.profiler.stop()
            if prev is not None:
                signal.signal(signal.SIGTERM, prev)
        return self.history

    def _should_exit(self) -> bool:
        """SIGTERM, ``exit_interval`` and ``exit_duration_in_mins`` (max-voted over ranks so all agree).
        Reference: mindspeed_mm/training.py:635-699."""
        cfg = self.cfg
        flag = self._sigterm
        if cfg.exit_interval and self.iteration % cfg.exit_interval == 0:
            flag = True
        if cfg.exit_duration_in_mins and (time.time() - self._t_start) / 60.0 > cfg.exit_duration_in_mins:
            flag = True
        if dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([int(flag)], device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            flag = bool(t.item())
        return flag

    @torch.no_grad()
    def validate(self) -> Optional[float]:
        tot, n = 0.0, 0
        for i, mb in enumerate(self.val_iter_fn()):
            if self.cfg.val_iters and i >= self.cfg.val_iters:
                break
            mb = to_device(mb, self.device) if self.device.type == "cuda" else mb
            out = self.model(mb, run=self.engine.run)
            loss = self.loss_fn(out[0], out[1]) if isinstance(out, tuple) else out
            tot += float(loss)
            n += 1
        if n == 0:
            return None
        val = torch.tensor(tot / n, device=self.device)
        if self.dp_world > 1:
            dist.all_reduce(val, group=self.dp_group)
            val /= self.dp_world
        print_rank0(f" ** validation after iteration {self.iteration} ** | validation steps: {n} |"
                    f" validation loss: {val.item():.6E} |")
        return float(val)

    # ---------------------------------------------------------------------------------- state
    def extra_state(self) -> dict:
        return dict(iteration=self.iteration, consumed_train_samples=self.consumed_train_samples,
                    lr_scheduler=self.schedule.state_dict(), torch_rng=torch.get_rng_state(),
                    cuda_rng=torch.cuda.get_rng_state() if self.device.type == "cuda" else None,
                    dataloader=getattr(self.data_iter, "state_dict", lambda: None)(),
                    ema=self.ema.state_dict() if self.ema is not None else None)

    def load_extra_state(self, s: dict, load_rng: bool = True) -> None:
        self.iteration = s["iteration"]
        self.consumed_train_samples = s["consumed_train_samples"]
        self.schedule.load_state_dict(s["lr_scheduler"])
        if load_rng:
            torch.set_rng_state(s["torch_rng"])
            if s.get("cuda_rng") is not None and self.device.type == "cuda":
                torch.cuda.set_rng_state(s["cuda_rng"])
        if s.get("dataloader") is not None and hasattr(self.data_iter, "load_state_dict"):
            self.data_iter.load_state_dict(s["dataloader"])
        if s.get("ema") is not None and self.ema is not None:
            self.ema.load_state_dict(s["ema"])

    def save(self):
        self.checkpointer.save(self.iteration, self.engine, self.extra_state())

    def load(self, **kw) -> bool:
        s = self.checkpointer.load(self.engine, **kw)
        if s is not None:
            self.load_extra_state(s, load_rng=kw.get("load_rng", True))
        return s is not None
