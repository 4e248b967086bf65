"""Debugging and planning helpers: a gradient probe, named timers, and a parallel-plan suggester.

* ``grad_probe(x, tag)`` -- identity in forward; in backward reports shape / sum / norm / max / non-finite count of the
  gradient that flows through ``x`` on the chosen rank, into the log and into ``PROBE_LOG`` (reference:
  mindspeed_mm/fsdp/tools/debug.py:5-86 ``DebugBwd`` / ``debug_fn``).
* ``Timers`` -- named interval timers with CUDA-event timing on the launching stream when a GPU is present; ``log()``
  gives the max over ranks and the Megatron-style ``name: ms | name: ms`` line (mindspeed_mm/training.py:896-920).
* ``suggest_parallel_plan`` -- enumerates (shard, ulysses, tensor, pipeline) splits of a GPU count, drops the ones whose
  memory model does not fit, and orders the rest by a time model of compute + exposed communication (the reference
  searches by timing short runs: mindspeed_mm/utils/auto_setting.py:67-170; here the search is analytic and the caller
  times the top few candidates).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .logging import get_logger
from .tools import estimate_training_memory

PROBE_LOG: List[dict] = []


class _GradProbe(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tag, rank, keep_value):
        ctx.tag, ctx.rank = tag, rank
        ctx.value = x.detach() if keep_value else None
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        me = dist.get_rank() if dist.is_initialized() else 0
        if ctx.rank < 0 or ctx.rank == me:
            gf = g.detach().float()
            rec = {"tag": ctx.tag, "rank": me, "shape": tuple(g.shape), "sum": float(gf.sum()), "norm": float(gf.norm()),
                   "absmax": float(gf.abs().max()) if gf.numel() else 0.0, "nonfinite": int((~torch.isfinite(gf)).sum())}
            if ctx.value is not None:
                rec["value_norm"] = float(ctx.value.float().norm())
            PROBE_LOG.append(rec)
            get_logger().info("[grad_probe] {tag} | shape={shape} | grad_sum={sum:.6f} | norm={norm:.6f} | absmax={absmax:.6f} "
                              "| nonfinite={nonfinite}".format(**rec))
        return g, None, None, None


def grad_probe(x: torch.Tensor, tag: str = "", rank: int = 0, keep_value: bool = False) -> torch.Tensor:
    """``x = grad_probe(x, "block3.out")`` anywhere in a model; ``rank=-1`` reports on every rank."""
    return _GradProbe.apply(x, tag, rank, keep_value)


# ------------------------------------------------------------------------------------------------- timers
class _Timer:
    def __init__(self, name: str, cuda: bool):
        self.name, self.cuda = name, cuda
        self.total_ms, self.count = 0.0, 0
        self._t0 = None
        self._pending = []

    def start(self):
        if self._t0 is not None:
            raise RuntimeError(f"timer {self.name!r} already started")
        if self.cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self):
        if self._t0 is None:
            raise RuntimeError(f"timer {self.name!r} was not started")
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pending.append((self._t0, e))          # read later: no synchronisation inside the step
        else:
            self.total_ms += (time.perf_counter() - self._t0) * 1e3
        self.count += 1
        self._t0 = None

    def elapsed(self, reset: bool = True) -> float:
        for a, b in self._pending:
            b.synchronize()
            self.total_ms += a.elapsed_time(b)
        self._pending = []
        v = self.total_ms
        if reset:
            self.total_ms, self.count = 0.0, 0
        return v

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()


class Timers:
    def __init__(self, cuda: Optional[bool] = None):
        self.cuda = torch.cuda.is_available() if cuda is None else cuda
        self._timers: Dict[str, _Timer] = {}

    def __call__(self, name: str) -> _Timer:
        if name not in self._timers:
            self._timers[name] = _Timer(name, self.cuda)
        return self._timers[name]

    def log(self, names: Optional[Sequence[str]] = None, normalizer: float = 1.0, reset: bool = True) -> str:
        """Max over ranks of every timer (ms / normalizer) as one line; rank 0 also writes it to the log."""
        names = list(names or self._timers)
        vals = torch.tensor([self._timers[n].elapsed(reset) / normalizer if n in self._timers else 0.0 for n in names],
                            dtype=torch.float64)
        if dist.is_initialized() and dist.get_world_size() > 1:
            if dist.get_backend() == "nccl":
                vals = vals.cuda()
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        line = "time (ms) | " + " | ".join(f"{n}: {v:.2f}" for n, v in zip(names, vals.tolist()))
        if not dist.is_initialized() or dist.get_rank() == 0:
            get_logger().info(line)
        return line


# ------------------------------------------------------------------------------------------------- plan search
@dataclass
class ModelShape:
    n_params: float
    n_layers: int
    hidden: int
    seq_len: int                      # tokens per sample (per data-parallel rank and micro-batch)
    heads: int = 32
    activation_bytes_per_token_layer: float = 34.0     # x hidden: saved tensors of one transformer layer in bf16
    flops_per_token: Optional[float] = None            # default 6 N (+ attention)


@dataclass
class Hardware:
    n_gpus: int = 8
    mem_gb: float = 180.0
    tflops: float = 1400.0            # sustained dense bf16
    link_gbs: float = 770.0           # per direction per GPU


def suggest_parallel_plan(model: ModelShape, hw: Hardware = Hardware(), recompute: bool = True, top: int = 5) -> List[dict]:
    """Candidates ``{"shard", "ulysses", "tp", "pp", "dp", "mem_gb", "step_ms", ...}`` sorted by modelled step time."""
    out = []
    n = hw.n_gpus
    divs = [d for d in range(1, n + 1) if n % d == 0]
    per_layer_act = model.activation_bytes_per_token_layer * model.hidden
    flops_tok = model.flops_per_token or (6.0 * model.n_params + 12.0 * model.n_layers * model.hidden * model.seq_len)
    for tp in divs:
        for pp in [d for d in divs if (n // tp) % d == 0 and model.n_layers % d == 0]:
            rest = n // tp // pp
            for uly in [d for d in divs if rest % d == 0 and model.heads % (d * tp) == 0]:
                dp = rest // uly
                shard = rest                                           # ZeRO-3 shards over data x sequence ranks
                tokens = model.seq_len / uly
                layers_here = model.n_layers // pp
                mem = estimate_training_memory(
                    model.n_params / pp, shard_world=shard, tp=tp, n_layers=layers_here,
                    recompute_layers=layers_here if recompute else 0,
                    activation_bytes_per_layer=per_layer_act * tokens / tp,
                    layer_input_bytes=2.0 * model.hidden * tokens,
                    largest_unit_params=model.n_params / model.n_layers)
                if mem["total_gb"] > hw.mem_gb:
                    continue
                compute = flops_tok * (4.0 / 3.0 if recompute else 1.0) * model.seq_len / (uly * tp) / pp / (hw.tflops * 1e12)
                p_bytes = 2.0 * model.n_params / pp / tp
                zero = (3.0 if recompute else 2.0) * p_bytes * (shard - 1) / shard + p_bytes * (shard - 1) / shard   # gathers + reduce-scatter
                a2a = 0.0 if uly == 1 else 4 * 2 * (3 if recompute else 2) * layers_here * tokens * model.hidden * 2 / tp * (uly - 1) / uly
                tpc = 0.0 if tp == 1 else 4 * (3 if recompute else 2) * layers_here * tokens * model.hidden * 2 * (tp - 1) / tp
                comm = (zero + a2a + tpc) / (hw.link_gbs * 1e9)
                exposed = max(0.0, zero / (hw.link_gbs * 1e9) - 0.8 * compute) + (a2a + tpc) / (hw.link_gbs * 1e9)
                bubble = (pp - 1) / (pp - 1 + max(dp, 1) * 4) if pp > 1 else 0.0     # 4 micro-batches per data rank assumed
                step = (compute + exposed) / (1.0 - bubble)
                out.append(dict(shard=shard, ulysses=uly, tp=tp, pp=pp, dp=dp, mem_gb=round(mem["total_gb"], 1),
                                compute_ms=round(compute * 1e3, 2), comm_ms=round(comm * 1e3, 2),
                                exposed_comm_ms=round(exposed * 1e3, 2), bubble=round(bubble, 3), step_ms=round(step * 1e3, 2),
                                samples_per_s=round(dp / step, 3) if step > 0 else math.inf))
    out.sort(key=lambda r: -r["samples_per_s"])
    return out[:top]
