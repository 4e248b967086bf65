"""Flat-buffer ZeRO-3 engine ("FSDP2" semantics without DTensor hooks).

What the reference gets from ``torch.distributed.fsdp.fully_shard`` plus its own hook
re-implementation (mindspeed_mm/fsdp/distributed/fully_shard_parallel.py:42-516,
mindspeed_mm/fsdp/ops/fully_shard/fully_shard.py:481-825) is here one small engine that
owns the memory layout, because the layout is what lets the collectives be fused:

* Every *unit* (a transformer layer, the embedding, the head ...) keeps its parameters in ONE
  contiguous bf16 buffer.  Rank r owns the r-th 1/world slice of it (``shard16``), plus the
  fp32 master copy and Adam moments of that slice only.
* ``unshard``   = all-gather of ``shard16`` into the full buffer (prefetched one unit ahead on
  a side stream).  On the native tier the gather is a kernel that pulls peer slices over
  NVLink from symmetric memory (see ``comm/symm.py``); otherwise NCCL/gloo.
* A unit runs as one autograd node that keeps only its inputs (activation checkpointing);
  backward re-gathers, recomputes, and then *reduce-scatters the bf16 gradients, casts to
  fp32 and applies sharded AdamW in one pass*, overlapped with the backward of the next unit.
  With gradient clipping or accumulation the update is deferred: the reduced fp32 gradient
  slice is kept and ``finish_step`` applies the update once the global norm is known.
* world == 1 degenerates to: persistent bf16 parameters, fused optimizer-in-backward.

Mixed precision follows ``param_dtype`` (compute / gather dtype) and ``reduce_dtype``
(gradient accumulation dtype), the two knobs of the reference's ``FSDPPlanConfig``
(mindspeed_mm/fsdp/params/parallel_args.py:13-35).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops

import os as _os
# diagnostic switch: the compute stream waits for each unit's reduce(+update) instead of overlapping with it
_SERIAL_REDUCE = _os.environ.get("MM_B200_SERIAL_REDUCE", "0") == "1"

ALIGN = 128  # elements; keeps every parameter 256-byte aligned inside the flat buffer (TMA needs 16 B)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class OptimConfig:
    lr: float = 1e-4
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    clip_grad: float = 0.0
    # parameter-name predicates: no weight decay for 1-D tensors and biases by default
    no_decay: Callable[[str, torch.Tensor], bool] = staticmethod(lambda n, p: p.dim() < 2 or n.endswith(".bias"))
    # "muon": 2-D hidden matrices take momentum + Newton-Schulz orthogonalisation, everything else AdamW
    # (fsdp/optimizer/optimizer.py:158-197 of the reference picks the same split)
    kind: str = "adamw"
    muon_momentum: float = 0.95
    ns_steps: int = 5
    matched_adamw_rms: float = 0.2
    muon_eligible: Callable[[str, torch.Tensor], bool] = staticmethod(
        lambda n, p: p.dim() == 2 and not n.endswith(".bias") and "embed" not in n and "lm_head" not in n
        and "output_layer" not in n)
    # per-parameter learning-rate multipliers: the first (regex, scale) whose regex matches the start of the parameter
    # name wins (``lr_scaling_plan`` of the reference, fsdp/optimizer/optimizer.py:310-331); recipes written against
    # Hugging Face module trees say ``model.visual...``, so the name is tried with that prefix too
    lr_scaling: Sequence[Tuple[str, float]] = ()
    # > 0: adaptive clipping (the reference's adaptive_clip_grad_norm patch): the threshold follows an exponential moving
    # average of the gradient norm plus three standard deviations instead of the fixed ``clip_grad``
    clip_grad_ema_decay: float = 0.0

    def lr_scale_of(self, name: str) -> float:
        import re
        for pat, scale in self.lr_scaling:
            if re.match(pat, name) or re.match(pat, "model." + name):
                return float(scale)
        return 1.0


def _sq_norm(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """Sum of squares over the fp32 gradient shards: one kernel per shard into a table of block partials and a single
    reduction on CUDA (fixed summation order), stacked reductions elsewhere."""
    from .. import ops
    if ops._native(tensors[0]) and all(t.dtype == torch.float32 for t in tensors):
        return ops._nat().sq_norm(tensors)
    return torch.stack([t.float().pow(2).sum() for t in tensors]).sum()


class ExtremeGradientError(RuntimeError):
    """Adaptive clipping met a gradient norm beyond ``max(mean + 5 sigma, 5)`` or a non-finite one: the step was not
    applied (mindspeed_mm/patchs/adaptive_clip_grad_patch.py:228-262 stops the run the same way)."""


class AdaptiveClip:
    """Threshold = moving average of the unclipped gradient norms + 3 sigma.  Norms under the threshold update the average
    and its variance and pass unclipped; norms above it (up to the extreme threshold) are scaled down to it and leave the
    statistics alone.  First step: average = min(3 * norm, 1), variance 0, no clipping."""

    def __init__(self, decay: float):
        self.decay, self.avg, self.var = decay, None, 0.0
        self.threshold = self.coef = None

    def scale_for(self, norm: float) -> float:
        import math
        if not math.isfinite(norm):
            raise ExtremeGradientError(f"gradient norm is {norm}")
        if self.avg is None:
            self.avg, self.var = min(3.0 * norm, 1.0), 0.0
            self.threshold, self.coef = self.avg, 1.0
            return 1.0
        thr = self.avg + 3.0 * self.var ** 0.5
        extreme = max(self.avg + 5.0 * self.var ** 0.5, 5.0)
        self.threshold = thr
        if norm <= thr:
            d = self.decay
            self.avg = d * self.avg + (1 - d) * norm
            self.var = d * self.var + (1 - d) * (self.avg - norm) ** 2
            self.coef = 1.0
        elif norm <= extreme:
            self.coef = thr / norm
        else:
            raise ExtremeGradientError(f"gradient norm {norm:.4g} is beyond the extreme threshold {extreme:.4g} "
                                       f"(moving average {self.avg:.4g}, variance {self.var:.4g})")
        return self.coef

    def state_dict(self):
        return dict(avg=self.avg, var=self.var)

    def load_state_dict(self, sd):
        self.avg, self.var = sd["avg"], sd["var"]


class FlatGroup:
    """One flat bf16 buffer + its sharded optimizer state."""

    def __init__(self, named_params: List[Tuple[str, nn.Parameter]], rank: int, world: int, device,
                 param_dtype: torch.dtype, trainable: bool, opt: OptimConfig, lr_scale: float = 1.0):
        self.rank, self.world, self.device = rank, world, device
        self.dtype = param_dtype
        self.trainable = trainable
        self.lr_scale = lr_scale
        # decayed parameters first so that weight decay is one split point in the flat index space; with Muon the
        # orthogonalised matrices come first of all, so that they are one prefix [0, muon_end) as well
        decay = [(n, p) for n, p in named_params if not (trainable and opt.no_decay(n, p))]
        nodecay = [(n, p) for n, p in named_params if (trainable and opt.no_decay(n, p))]
        n_muon = 0
        if trainable and opt.kind == "muon":
            mu = [(n, p) for n, p in decay if opt.muon_eligible(n, p)]
            decay = mu + [(n, p) for n, p in decay if not opt.muon_eligible(n, p)]
            n_muon = len(mu)
        self.named_params = decay + nodecay
        self.shapes: List[torch.Size] = [p.shape for _, p in self.named_params]
        self.numels: List[int] = [p.numel() for _, p in self.named_params]
        self.offsets: List[int] = []
        off = 0
        for i, (n, p) in enumerate(self.named_params):
            if i == len(decay):
                self.decay_end = off
            self.offsets.append(off)
            off = _round_up(off + p.numel(), ALIGN)
        if not nodecay:
            self.decay_end = off
        self.n_muon = n_muon
        self.muon_end = self.offsets[n_muon] if n_muon < len(self.offsets) else off
        self.numel = off
        self.padded = _round_up(max(off, 1), world * ALIGN)
        self.shard_numel = self.padded // world
        self.full: Optional[torch.Tensor] = None          # [padded] when unsharded
        self.shard16: Optional[torch.Tensor] = None       # [shard_numel]
        self.master = self.exp_avg = self.exp_avg_sq = None
        self.grad32: Optional[torch.Tensor] = None        # deferred-update accumulator
        self.symm = None                                   # symmetric-memory handle of shard16 (native tier)
        self.step_count = 0

    # ---- memory ---------------------------------------------------------------------------
    def alloc_full(self) -> torch.Tensor:
        if self.world == 1:
            return self.shard16
        return torch.empty(self.padded, dtype=self.dtype, device=self.device)

    def bind(self, full: torch.Tensor) -> None:
        """Point every parameter at its view of ``full``."""
        self.full = full
        for (n, p), off, shape, numel in zip(self.named_params, self.offsets, self.shapes, self.numels):
            p.data = full[off:off + numel].view(shape)

    def release(self) -> None:
        if self.world == 1:
            return
        self.full = None
        for _, p in self.named_params:
            p.data = _EMPTY[self.device, self.dtype]

    def local_slice(self, flat: torch.Tensor) -> torch.Tensor:
        return flat[self.rank * self.shard_numel:(self.rank + 1) * self.shard_numel]

    def init_state(self) -> None:
        """Called once with ``full`` bound and initialised: carve this rank's persistent state."""
        src = self.local_slice(self.full)
        if self.world == 1:
            self.shard16 = self.full
        else:
            self.shard16 = src.clone()
        if self.trainable:
            self.master = src.float()
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)

    def flat_grads(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Copy the parameters' ``.grad`` into one flat buffer (pads zero) and drop the originals."""
        g = out if out is not None else torch.empty(self.padded, dtype=self.dtype, device=self.device)
        views, srcs, prev_end = [], [], 0
        base, esz = g.data_ptr(), g.element_size()
        for (n, p), off, shape, numel in zip(self.named_params, self.offsets, self.shapes, self.numels):
            if off > prev_end:
                g[prev_end:off].zero_()
            if p.grad is None:
                g[off:off + numel].zero_()
            elif p.grad.data_ptr() != base + off * esz or p.grad.dtype != g.dtype:
                views.append(g[off:off + numel].view(shape))
                srcs.append(p.grad)
            # else: the weight-gradient GEMM already wrote this slice of the flat buffer (see offer_grad_buffer)
            prev_end = off + numel
        if prev_end < self.padded:
            g[prev_end:].zero_()
        if views:
            torch._foreach_copy_(views, srcs)
        for _, p in self.named_params:
            p.grad = None
            p._grad_flat = None
        return g

    def offer_grad_buffer(self, flat: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Allocate this group's flat gradient buffer BEFORE the unit's backward and tell every parameter where its
        slice lives, so that a weight-gradient GEMM can write there directly (``ops.native._Linear.backward``);
        ``flat_grads(out=buffer)`` then skips the copy for the slices that were filled in place."""
        if flat is None:
            flat = torch.empty(self.padded, dtype=self.dtype, device=self.device)
        for (n, p), off, shape, numel in zip(self.named_params, self.offsets, self.shapes, self.numels):
            p._grad_flat = (flat, off, numel, shape) if p.requires_grad else None
        return flat


class _Empty(dict):
    def __missing__(self, key):
        dev, dt = key
        self[key] = torch.empty(0, dtype=dt, device=dev)
        return self[key]


_EMPTY = _Empty()


class Unit:
    def __init__(self, name: str, module: nn.Module, engine: "FSDPEngine"):
        self.name, self.module, self.engine = name, module, engine
        named = [(f"{name}.{n}" if name else n, p) for n, p in module.named_parameters()
                 if id(p) not in engine.exclude_params]
        train = [(n, p) for n, p in named if p.requires_grad]
        frozen = [(n, p) for n, p in named if not p.requires_grad]
        mk = lambda ps, tr, sc=1.0: FlatGroup(ps, engine.rank, engine.world, engine.device, engine.param_dtype, tr,
                                              engine.opt, sc)
        by_scale: Dict[float, list] = {}
        for n, p in train:                  # one flat group per learning-rate multiplier (usually just one)
            by_scale.setdefault(engine.opt.lr_scale_of(n), []).append((n, p))
        self.groups: List[FlatGroup] = [mk(ps, True, sc) for sc, ps in by_scale.items()] + \
            ([mk(frozen, False)] if frozen else [])
        # shapes are recorded by the groups above; now swap in re-bindable placeholders
        mapping = _to_flat_params(module, engine.device, engine.param_dtype, engine.exclude_params)
        for g in self.groups:
            g.named_params = [(n, mapping[id(p)]) for n, p in g.named_params]
        self.unsharded = False
        self.ready_event = None
        self.index = -1
        self.bwd_done = False          # backward of the current micro-step has run
        self.recompute = True          # False: keep the autograd graph (used for the loss head)
        self.pending_reduce = False    # non-recompute unit whose gradients wait to be reduced
        # a unit may run more than once per micro-batch (an embedding or output head shared with a multi-token-prediction
        # block): its gradients are reduced after the LAST of its backward passes
        self.uses = 0                  # differentiated forward calls in this micro-batch
        self.bwd_uses = 0              # backward passes seen so far
        self.hooks = 0                 # completion hooks registered (graph-keeping units with a differentiable input)
        # what the engine calls to run the unit: the module itself, or (models whose own forward has been re-routed
        # through ``engine.run``, see plugins/hf_adapter.py) the class-level forward that the re-routing bypasses
        self.call = None

    def invoke(self, *args, **kwargs):
        return self.module(*args, **kwargs) if self.call is None else self.call(*args, **kwargs)

    @property
    def trainable(self):
        return any(g.trainable for g in self.groups)


class FSDPEngine:
    """Shards ``units`` over ``group`` and runs them with gather / recompute / reduce+update."""

    def __init__(self, units: Sequence[Tuple[str, nn.Module]], group: Optional[dist.ProcessGroup] = None,
                 device: torch.device | str = "cpu", param_dtype: torch.dtype = torch.bfloat16,
                 reduce_dtype: torch.dtype = torch.float32, opt: Optional[OptimConfig] = None,
                 recompute: bool = True, grad_accum_steps: int = 1, prefetch: int = 1,
                 comm: str = "auto", grad_divide: Optional[float] = None,
                 no_recompute: Sequence[str] = ("lm_head",), exclude_params: Sequence[nn.Parameter] = (),
                 replicate_group: Optional[dist.ProcessGroup] = None, offload_optimizer: bool = False):
        """``replicate_group`` (hybrid sharding, HSDP): parameters are sharded over ``group`` and replicated over
        ``replicate_group``; gradients are reduce-scattered inside the shard group and the reduced fp32 shard is then
        all-reduced across the replicas before the update (fsdp/distributed/fully_shard_parallel.py:42-109 on a 2-D
        mesh).  ``offload_optimizer``: fp32 master weights and Adam moments live in pinned host memory and visit the
        device one flat group at a time for the update (the reference's ``offload_to_cpu`` / CPUOffloadPolicy)."""
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and group is not False) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.device = torch.device(device)
        self.param_dtype, self.reduce_dtype = param_dtype, reduce_dtype
        self.opt = opt or OptimConfig()
        self.recompute = recompute
        self.grad_accum_steps = grad_accum_steps
        self.prefetch = prefetch
        self.reshard_after_forward = True     # False: a unit stays gathered between its forward and its backward
        self.activation_offload = None        # runtime.features.ActivationOffload for the units in _offload_units
        self._offload_units: set = set()
        self.replicate_group = replicate_group
        self.replicas = dist.get_world_size(replicate_group) if replicate_group is not None else 1
        self.offload_optimizer = offload_optimizer
        self.grad_divide = float(grad_divide if grad_divide is not None else self.world * self.replicas)
        self.exclude_params = {id(p) for p in exclude_params}    # owned by another engine (e.g. experts)
        self.units: List[Unit] = [Unit(n, m, self) for n, m in units]
        for i, u in enumerate(self.units):
            u.index = i
            u.recompute = recompute and u.name not in no_recompute
        self._by_module: Dict[int, Unit] = {id(u.module): u for u in self.units}
        self.cuda = self.device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.micro_step = 0
        self.lr = self.opt.lr
        # replicas and host-resident optimizer state both need the reduced gradient shard before the update runs
        self.adaptive_clip = AdaptiveClip(self.opt.clip_grad_ema_decay) if self.opt.clip_grad_ema_decay > 0 else None
        self.deferred = self.opt.clip_grad > 0 or grad_accum_steps > 1 or self.replicas > 1 or offload_optimizer or \
            self.opt.kind == "muon" or self.adaptive_clip is not None
        self._sq_norm = torch.zeros((), dtype=torch.float32, device=self.device)
        self._dummy = torch.zeros((), device=self.device, requires_grad=True)
        self.comm = comm
        self._p2p = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.kernel_launches = 0
        self._exec_order: List[Unit] = []
        self._exec_pos: Dict[int, int] = {}
        self._order_known = False

    # ------------------------------------------------------------------ materialisation
    def materialize(self, init_fn: Callable[[str, nn.Module], None]) -> None:
        """Allocate, initialise (``init_fn(unit_name, module)`` with full params bound) and shard."""
        for u in self.units:
            for g in u.groups:
                g.bind(torch.zeros(g.padded, dtype=g.dtype, device=g.device))
            init_fn(u.name, u.module)
            for g in u.groups:
                g.init_state()
                if self.offload_optimizer and g.trainable:
                    pin = self.cuda
                    g.master, g.exp_avg, g.exp_avg_sq = (
                        (t.cpu().pin_memory() if pin else t.cpu()) for t in (g.master, g.exp_avg, g.exp_avg_sq))
                if g.world > 1:
                    g.release()
            u.unsharded = self.world == 1
        self._setup_comm()

    def _setup_comm(self):
        if self.world > 1 and self.cuda and self.comm in ("auto", "p2p"):
            try:
                from ..comm.symm import P2PCollectives
                self._p2p = P2PCollectives(self)
            except Exception as e:  # noqa: BLE001
                if self.comm == "p2p":
                    raise
                self._p2p = None
                self._p2p_why = repr(e)

    # ------------------------------------------------------------------ gather / release
    def unshard(self, u: Unit, async_op: bool = True) -> None:
        if u.unsharded:
            return
        u.unsharded = True
        fulls = [g.alloc_full() for g in u.groups]
        if self.cuda:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                for g, f in zip(u.groups, fulls):
                    self._all_gather(g, f)
                    if self.world > 1:
                        f.record_stream(self.comm_stream)
                u.ready_event = torch.cuda.Event()
                u.ready_event.record()
        else:
            for g, f in zip(u.groups, fulls):
                self._all_gather(g, f)
        for g, f in zip(u.groups, fulls):
            g.bind(f)

    def wait_unshard(self, u: Unit) -> None:
        if u.ready_event is not None:
            torch.cuda.current_stream().wait_event(u.ready_event)
            u.ready_event = None

    def reshard(self, u: Unit, force: bool = False) -> None:
        if self.world == 1 or not u.unsharded:
            return
        if getattr(u, "keep_gathered", False) and not force:
            return          # "root" parameters: gathered once per micro-step, released in end_micro_step
        for g in u.groups:
            g.release()
        u.unsharded = False

    def _all_gather(self, g: FlatGroup, full: torch.Tensor) -> None:
        if self._p2p is not None:
            self._p2p.all_gather(g, full)
        else:
            dist.all_gather_into_tensor(full, g.shard16, group=self.group)

    # ------------------------------------------------------------------ running a unit
    def run(self, module: nn.Module, *args, **kwargs):
        """Execute ``module(*args)`` as a sharded, checkpointed unit."""
        u = self._by_module.get(id(module))
        if u is None:
            return module(*args, **kwargs)
        if not torch.is_grad_enabled():
            self.unshard(u)
            self.wait_unshard(u)
            self._prefetch_forward(u)
            out = u.invoke(*args, **kwargs)
            self.reshard(u)
            return out
        u.uses += 1
        if not u.recompute:
            # Plain autograd through the unit (its graph is kept).  Its gradients are complete once any
            # earlier unit starts its backward (or at finish_step), which is where they are reduced.
            self.unshard(u)
            self.wait_unshard(u)
            self._prefetch_forward(u)
            u.pending_reduce = u.trainable
            if u.trainable:
                self._hook_backward_done(u, args, kwargs)
            out = u.invoke(*args, **kwargs)
            if u.trainable and self.cuda and self._p2p is None:
                # offer the flat gradient buffer when this unit's backward is about to start (its output gradient
                # exists); with peer-memory slots the buffer is taken late instead, so that a slot is not held while
                # the previous unit's reduce-scatter is still reading the other one
                first = next((t for t in (out if isinstance(out, (tuple, list)) else (out,))
                              if isinstance(t, torch.Tensor) and t.requires_grad), None)
                if first is not None:
                    first.register_hook(lambda g, u=u: self._offer_buffers(u))
            return out
        tensors, spec = _split_args(args, kwargs)
        if self.activation_offload is not None and u.name in self._offload_units:
            with self.activation_offload:         # the unit's saved inputs go to pinned host memory until its backward
                outs = _UnitFn.apply(self, u, spec, self._dummy, *tensors)
        else:
            outs = _UnitFn.apply(self, u, spec, self._dummy, *tensors)
        return outs[0] if len(outs) == 1 and not u._tuple_out else outs

    def _prefetch_forward(self, u: Unit):
        """Gather the unit(s) that ran after ``u`` in the recorded forward order (none until one full
        forward has been seen: the order is learnt, not assumed from the list)."""
        if not self._order_known:
            if not self._exec_order or self._exec_order[-1] is not u:
                self._exec_order.append(u)
            return
        pos = self._exec_pos.get(id(u))
        if pos is None:
            return
        for k in range(1, self.prefetch + 1):
            if pos + k < len(self._exec_order):
                self.unshard(self._exec_order[pos + k])

    def _prefetch_backward(self, u: Unit):
        """Backward visits units in (roughly) reverse forward order; a unit prefetched too early or twice
        is harmless because everything still gathered is released in ``finish_step``."""
        if not self._order_known:
            return
        pos = self._exec_pos.get(id(u))
        if pos is None:
            return
        for k in range(1, self.prefetch + 1):
            if pos - k >= 0 and not self._exec_order[pos - k].bwd_done:
                self.unshard(self._exec_order[pos - k])

    def _seal_order(self):
        if not self._order_known and self._exec_order:
            self._order_known = True
            self._exec_pos = {id(u): i for i, u in enumerate(self._exec_order)}

    # ------------------------------------------------------------------ gradient reduce + update
    def _hook_backward_done(self, u: Unit, args, kwargs) -> None:
        """A unit that keeps its graph has finished its backward once the gradient of its (first differentiable)
        input exists.  Its reduce + update is issued when the *next* unit reports done (one unit of slack, so a
        weight-gradient node scheduled after the input gradient cannot be missed); the last one is picked up by
        ``flush_pending``.  Units without a differentiable input are reduced by ``flush_pending`` only."""
        for t in list(args) + list(kwargs.values()):
            if isinstance(t, torch.Tensor) and t.requires_grad:
                u.hooks += 1
                t.register_hook(lambda g, u=u: self._unit_backward_done(u))
                return

    def _offer_buffers(self, u: Unit) -> None:
        if u.bwd_uses:                 # a later use of a shared unit: its gradients accumulate into the buffers already offered
            return
        u._offered = {id(g): g.offer_grad_buffer() for g in u.groups if g.trainable}

    def _unit_backward_done(self, u: Unit) -> None:
        u.bwd_uses += 1
        prev = getattr(self, "_done_wait", None)
        if prev is not None and prev is not u and prev.pending_reduce:
            self._reduce_pending(prev)
            self._done_wait = None
        if u.bwd_uses >= u.hooks:          # every differentiated call of the unit has finished its backward
            self._done_wait = u

    def _reduce_pending(self, u: Unit) -> None:
        u.pending_reduce = False
        u.bwd_done = True
        if any(p.grad is not None for g in u.groups for _, p in g.named_params):
            self.reduce_and_update(u)
        self.reshard(u)

    def flush_pending(self, after: Optional[Unit] = None) -> None:
        """Reduce every graph-keeping unit whose backward is over: all of them (``after`` None, end of the step) or
        those that ran after ``after`` in the forward (their backward precedes ``after``'s)."""
        pos = self._exec_pos if self._order_known else {id(u): i for i, u in enumerate(self.units)}
        lo = pos.get(id(after), -1) if after is not None else -1
        for u in self.units:
            if u.pending_reduce and pos.get(id(u), 1 << 30) > lo and (after is None or u.bwd_uses >= u.hooks):
                self._reduce_pending(u)
        if after is None:
            self._done_wait = None

    def reduce_and_update(self, u: Unit) -> None:
        last_micro = (self.micro_step + 1) % self.grad_accum_steps == 0
        for g in u.groups:
            if not g.trainable:
                continue
            for _, prm in g.named_params:          # sequence-parallel replicas saw only a slice of the tokens
                tpg = getattr(prm, "_tp_sum_group", None)
                if tpg is not None and prm.grad is not None:
                    dist.all_reduce(prm.grad, group=tpg)
            offered = getattr(u, "_offered", None)
            buf = offered.pop(id(g), None) if offered else None
            if buf is None and self._p2p is not None:
                buf = self._p2p.grad_slot(g)
            flat = g.flat_grads(buf)
            if self.cuda:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                flat.record_stream(self.comm_stream)
                ctx = torch.cuda.stream(self.comm_stream)
            else:
                ctx = _null()
            with ctx:
                fused = not self.deferred and last_micro
                if self._p2p is not None:
                    self._p2p.reduce_scatter_update(g, flat, fused, self)
                else:
                    gshard = self._reduce_scatter(g, flat)
                    if fused:
                        self._adamw(g, gshard, 1.0 / self.grad_divide if self.world == 1 else 1.0)
                    else:
                        if g.grad32 is None:
                            g.grad32 = torch.zeros(g.shard_numel, dtype=self.reduce_dtype, device=self.device)
                        g.grad32.add_(gshard, alpha=1.0 / self.grad_divide if self.world == 1 else 1.0)
            if self.cuda and _SERIAL_REDUCE:
                torch.cuda.current_stream().wait_stream(self.comm_stream)

    def _reduce_scatter(self, g: FlatGroup, flat: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return flat
        src = flat.to(self.reduce_dtype)
        src.div_(self.grad_divide)
        out = torch.empty(g.shard_numel, dtype=self.reduce_dtype, device=self.device)
        dist.reduce_scatter_tensor(out, src, group=self.group)
        return out

    def _adamw(self, g: FlatGroup, grad: torch.Tensor, grad_scale, start: int = 0) -> None:
        """AdamW on this rank's shard of ``g`` from element ``start`` on (Muon owns the elements before it)."""
        if start == 0:
            g.step_count += 1
            if self.opt.kind == "muon" and g.muon_end > 0:
                return self._muon(g, grad, grad_scale)
        o = self.opt
        lr = self.lr * g.lr_scale
        lo = g.rank * g.shard_numel
        split = min(max(g.decay_end - lo, start), g.shard_numel)
        if start >= g.shard_numel:
            return
        if self.cuda and ops.get_tier() == "native":
            from ..ops import native
            native.adamw_shard(g.master[start:], g.exp_avg[start:], g.exp_avg_sq[start:], grad[start:], g.shard16[start:],
                               lr, o.betas[0], o.betas[1], o.eps, o.weight_decay, g.step_count, split - start, grad_scale)
            return
        if isinstance(grad_scale, torch.Tensor):
            grad = grad.float() * grad_scale
            grad_scale = 1.0
        for a, b, wd in ((start, split, o.weight_decay), (split, g.shard_numel, 0.0)):
            if b > a:
                ops.ref.adamw_step(g.master[a:b], g.exp_avg[a:b], g.exp_avg_sq[a:b], grad[a:b], lr, o.betas[0],
                                   o.betas[1], o.eps, wd, g.step_count, grad_scale, g.shard16[a:b])

    def _muon(self, g: FlatGroup, grad: torch.Tensor, grad_scale) -> None:
        """Muon on the matrices of ``g`` ([0, muon_end) of the flat index space), AdamW on the rest.

        The momentum lives in ``exp_avg`` of the owned slice.  Newton-Schulz needs whole matrices: the ranks all-gather
        the Nesterov-blended update, each orthogonalises the matrices it is assigned (round-robin), and a reduce-scatter
        of the (disjointly filled) result hands every rank its slice back - two collectives of the group's size per
        step, no redundant matrix work."""
        from ..runtime.optim_extra import newton_schulz
        o = self.opt
        lr = self.lr * g.lr_scale
        lo = g.rank * g.shard_numel
        b = min(max(g.muon_end - lo, 0), g.shard_numel)                     # my elements [0, b) belong to Muon matrices
        gs = grad.float() * grad_scale if (isinstance(grad_scale, torch.Tensor) or grad_scale != 1.0) else grad.float()
        upd = torch.zeros(g.shard_numel, dtype=torch.float32, device=self.device)
        if b:
            mom = g.exp_avg[:b]
            mom.mul_(o.muon_momentum).add_(gs[:b])
            upd[:b] = gs[:b] + o.muon_momentum * mom                      # Nesterov
        if self.world > 1:
            full = torch.empty(g.padded, dtype=torch.float32, device=self.device)
            dist.all_gather_into_tensor(full, upd, group=self.group)
        else:
            full = upd
        out = torch.zeros_like(full)
        for i in range(g.n_muon):
            if i % self.world != self.rank:
                continue
            off, shape = g.offsets[i], g.shapes[i]
            m = newton_schulz(full[off:off + g.numels[i]].view(shape), o.ns_steps)
            out[off:off + g.numels[i]] = (m * (o.matched_adamw_rms * max(shape) ** 0.5)).reshape(-1)
        if self.world > 1:
            mine = torch.empty(g.shard_numel, dtype=torch.float32, device=self.device)
            if self.cuda:
                dist.reduce_scatter_tensor(mine, out, group=self.group)
            else:                                                            # gloo has no reduce_scatter
                dist.all_reduce(out, group=self.group)
                mine.copy_(g.local_slice(out))
        else:
            mine = out
        if b:
            g.master[:b].mul_(1.0 - lr * o.weight_decay).add_(mine[:b], alpha=-lr)
            g.shard16[:b].copy_(g.master[:b])
        self._adamw(g, grad, grad_scale, start=b)

    def _adamw_offloaded(self, g: FlatGroup, grad: torch.Tensor, grad_scale) -> None:
        """Optimizer state on the host: bring master / moments of this group to the device, update, send them back."""
        host = (g.master, g.exp_avg, g.exp_avg_sq)
        g.master, g.exp_avg, g.exp_avg_sq = (t.to(self.device, non_blocking=True) for t in host)
        self._adamw(g, grad, grad_scale)
        for h, d in zip(host, (g.master, g.exp_avg, g.exp_avg_sq)):
            h.copy_(d, non_blocking=True)
        if self.cuda:
            torch.cuda.current_stream().synchronize()     # the device copies are dropped next: the host copies must be done
        g.master, g.exp_avg, g.exp_avg_sq = host

    def finish_step(self, lr: Optional[float] = None) -> Optional[torch.Tensor]:
        """Call after the last backward of an optimizer step.  Applies deferred updates (with the
        global-norm clip) and joins the side stream.  Returns the gradient norm when one was computed."""
        self.flush_pending()
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        if self._p2p is not None and not self.deferred:
            self._p2p.step_barrier()      # no rank gathers a shard before its owner finished updating it
        norm = None
        if self.deferred:
            groups = [g for u in self.units for g in u.groups if g.trainable and g.grad32 is not None]
            scale = 1.0
            if self.replicas > 1:       # HSDP: sum the shard over the replicas (the 1/N of all data ranks is in grad_divide)
                for g in groups:
                    dist.all_reduce(g.grad32, group=self.replicate_group)
            if self.opt.clip_grad > 0 or self.adaptive_clip is not None:
                sq = _sq_norm([g.grad32 for g in groups])
                if self.world > 1:
                    dist.all_reduce(sq, group=self.group)
                norm = sq.sqrt() / self.grad_accum_steps      # norm of the micro-batch-averaged gradient
                if self.adaptive_clip is not None:
                    try:
                        scale = self.adaptive_clip.scale_for(float(norm))     # the norm is the same on every rank
                    except ExtremeGradientError:
                        for g in groups:                                       # the step is not applied
                            g.grad32 = None
                        raise
                else:
                    scale = torch.clamp(self.opt.clip_grad / (norm + 1e-6), max=1.0)
            if self.grad_accum_steps > 1:
                scale = scale / self.grad_accum_steps
            for g in groups:
                if self.offload_optimizer:
                    self._adamw_offloaded(g, g.grad32, scale)
                else:
                    self._adamw(g, g.grad32, scale)
                g.grad32 = None
            if self._p2p is not None:
                self._p2p.step_barrier()
        self.last_grad_norm = norm
        return norm

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def select_units(self, apply_names: Optional[Sequence[str]] = None, reshard_after_forward: bool = True) -> None:
        """Sharding plan of the native schema.  ``apply_names``: units gathered and released one by one (the modules a
        recipe lists under ``fsdp_plan.apply_modules``); every other unit belongs to the "root" wrap: sharded as well,
        but gathered once per micro-step and released after the backward, like the parameters the reference leaves to
        the outer ``fully_shard(model)`` (fsdp/distributed/fully_shard_parallel.py:98-109).  ``reshard_after_forward``
        False keeps every unit gathered between forward and backward (no second gather, more memory)."""
        self.reshard_after_forward = reshard_after_forward
        if apply_names is not None:
            names = set(apply_names)
            for u in self.units:
                u.keep_gathered = u.name not in names

    def set_activation_offload(self, offload, unit_names: Sequence[str]) -> None:
        self.activation_offload, self._offload_units = offload, set(unit_names)

    def end_micro_step(self) -> None:
        """Call after each micro-batch's backward."""
        self.flush_pending()
        self._seal_order()
        for u in self.units:
            u.bwd_done = False
            u.uses = u.bwd_uses = u.hooks = 0
            self.reshard(u, force=True)       # anything a prefetch gathered but nobody consumed, and the root units
        self.micro_step += 1

    # ------------------------------------------------------------------ state
    def named_full_params(self) -> Iterable[Tuple[str, torch.Tensor]]:
        """Yield (name, full tensor) unit by unit (gathers; every rank must iterate)."""
        for u in self.units:
            was = u.unsharded
            self.unshard(u)
            self.wait_unshard(u)
            for g in u.groups:
                for n, p in g.named_params:
                    yield n, p.data
            if not was:
                self.reshard(u)

    def load_full_params(self, getter: Callable[[str, torch.Size], Optional[torch.Tensor]]) -> List[str]:
        """Fill parameters from ``getter(name, shape)``; returns the names that were missing."""
        missing = []
        for u in self.units:
            for g in u.groups:
                full = torch.zeros(g.padded, dtype=g.dtype, device=g.device) if self.world > 1 else g.shard16
                if self.world > 1:
                    self._all_gather(g, full)
                for (n, p), off, shape, numel in zip(g.named_params, g.offsets, g.shapes, g.numels):
                    t = getter(n, shape)
                    if t is None:
                        missing.append(n)
                        continue
                    full[off:off + numel].copy_(t.reshape(-1))
                src = g.local_slice(full)
                if self.world > 1:
                    g.shard16.copy_(src)
                if g.trainable:
                    g.master.copy_(src)
        self.sync_after_load()
        return missing

    def sync_after_load(self) -> None:
        """With peer-memory collectives the bf16 shards live in the symmetric arena and a peer's gather kernel reads
        them without any flag: after the shards were written from the host side (weight load, checkpoint load) every
        rank waits here until all ranks have finished writing, before anyone gathers."""
        if self._p2p is not None:
            self._p2p.sync_after_load()

    def sharded_state(self) -> dict:
        out = {}
        for u in self.units:
            for gi, g in enumerate(u.groups):
                k = f"{u.name}#{gi}"
                out[k] = dict(shard16=g.shard16, master=g.master, exp_avg=g.exp_avg, exp_avg_sq=g.exp_avg_sq,
                              step=g.step_count, world=self.world, rank=self.rank, numel=g.numel)
        return out

    def load_sharded_state(self, state: dict, load_optim: bool = True) -> None:
        for u in self.units:
            for gi, g in enumerate(u.groups):
                s = state[f"{u.name}#{gi}"]
                if s["world"] != self.world or s.get("rank", self.rank) != self.rank:
                    raise ValueError("sharded state was saved for another rank / size of the sharding group; "
                                     "load it through the checkpointer (it re-slices) or use the full format")
                g.shard16.copy_(s["shard16"])
                if g.trainable:
                    g.master.copy_(s["master"] if s.get("master") is not None else s["shard16"])
                    if load_optim and s.get("exp_avg") is not None:
                        g.exp_avg.copy_(s["exp_avg"])
                        g.exp_avg_sq.copy_(s["exp_avg_sq"])
                        g.step_count = s["step"]
        self.sync_after_load()

    def param_count(self) -> int:
        return sum(g.numel for u in self.units for g in u.groups)


def _to_flat_params(module: nn.Module, device, dtype, exclude=()) -> dict:
    """Swap every parameter for a same-shaped placeholder of the flat buffer's device/dtype.

    The placeholder's storage is replaced by a view of the flat buffer in ``FlatGroup.bind``; the
    parameter keeps reporting its logical shape only while bound, so shapes are recorded by the group.
    Works for modules built under ``torch.device("meta")`` (nothing is ever allocated for them).
    """
    mapping = {}
    for m in module.modules():
        for n, p in list(m._parameters.items()):
            if p is None or id(p) in exclude:
                continue
            if id(p) not in mapping:
                q = nn.Parameter(torch.empty(0, dtype=dtype, device=device), requires_grad=p.requires_grad)
                q.__dict__.update(p.__dict__)            # keep tags such as _tp_sum_group
                mapping[id(p)] = q
            m._parameters[n] = mapping[id(p)]
    return mapping


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _flatten_arg(a, tensors):
    """Replaces every tensor inside ``a`` (also inside dicts / lists / tuples) by its index into ``tensors``."""
    if isinstance(a, torch.Tensor):
        tensors.append(a)
        return ("t", len(tensors) - 1)
    if isinstance(a, dict):
        return ("d", {k: _flatten_arg(v, tensors) for k, v in a.items()})
    if isinstance(a, (list, tuple)) and any(isinstance(v, (torch.Tensor, dict, list, tuple)) for v in a):
        return ("l", type(a), [_flatten_arg(v, tensors) for v in a])
    return ("c", a)


def _unflatten_arg(spec, tensors):
    kind = spec[0]
    if kind == "t":
        return tensors[spec[1]]
    if kind == "c":
        return spec[1]
    if kind == "d":
        return {k: _unflatten_arg(v, tensors) for k, v in spec[1].items()}
    return spec[1](_unflatten_arg(v, tensors) for v in spec[2])


def _split_args(args, kwargs):
    tensors: list = []
    spec = [_flatten_arg(a, tensors) for a in args]
    kspec = {k: _flatten_arg(a, tensors) for k, a in kwargs.items()}
    return tensors, (spec, kspec)


def _join_args(spec, tensors):
    a_spec, k_spec = spec
    return [_unflatten_arg(v, tensors) for v in a_spec], {n: _unflatten_arg(v, tensors) for n, v in k_spec.items()}


class _UnitFn(torch.autograd.Function):
    """gather -> forward (no graph kept) -> release; backward: gather -> recompute -> grads ->
    reduce-scatter + optimizer -> release.  Holds only the unit's inputs between the two."""

    @staticmethod
    def forward(ctx, engine: FSDPEngine, u: Unit, spec, dummy, *tensors):
        ctx.engine, ctx.u, ctx.spec = engine, u, spec
        engine.unshard(u)
        engine.wait_unshard(u)
        engine._prefetch_forward(u)
        args, kwargs = _join_args(spec, tensors)
        ctx.act_cache = []
        with torch.no_grad(), ops.activation_cache(ctx.act_cache, "record"):
            out = u.invoke(*args, **kwargs)
        if engine.reshard_after_forward:
            engine.reshard(u)
        ctx.save_for_backward(*tensors)
        ctx.needs = [t.requires_grad for t in tensors]
        u._tuple_out = isinstance(out, (tuple, list))
        outs = tuple(out) if u._tuple_out else (out,)
        ctx.out_is_tensor = [isinstance(o, torch.Tensor) for o in outs]
        ctx.mark_non_differentiable(*[o for o in outs if isinstance(o, torch.Tensor) and not o.is_floating_point()])
        return outs

    @staticmethod
    def backward(ctx, *gouts):
        engine, u = ctx.engine, ctx.u
        tensors = [t.detach().requires_grad_(need) for t, need in zip(ctx.saved_tensors, ctx.needs)]
        u.bwd_uses += 1
        last = u.bwd_uses >= u.uses            # the unit ran more than once: reduce after its last backward
        engine.flush_pending(after=u)
        engine.unshard(u)
        engine.wait_unshard(u)
        engine._prefetch_backward(u)
        if u.trainable and engine.cuda and u.bwd_uses == 1:
            # with peer-memory collectives the buffer is the next gradient slot of the symmetric arena
            u._offered = {id(g): g.offer_grad_buffer(engine._p2p.grad_slot(g) if engine._p2p is not None else None)
                          for g in u.groups if g.trainable}
        args, kwargs = _join_args(ctx.spec, tensors)
        with torch.enable_grad(), ops.recompute_region(), ops.activation_cache(ctx.act_cache, "replay"):
            out = u.invoke(*args, **kwargs)
        ctx.act_cache = None
        outs = tuple(out) if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, gouts)
                 if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        if u.trainable and last:
            engine.reduce_and_update(u)
        engine.reshard(u)
        u.bwd_done = last
        grads = [t.grad if need else None for t, need in zip(tensors, ctx.needs)]
        return (None, None, None, None, *grads)


class EngineMux:
    """Two engines over one model: dense parameters (sharded over the FSDP group) and expert parameters
    (sharded over the expert-FSDP group, gradients divided by the full data-parallel size).  The reference
    builds the same split with a second ``fully_shard`` mesh and a second optimizer
    (fsdp/distributed/expert_parallel/expert_fully_shard_parallel.py:22-57, fsdp/optimizer/optimizer.py:374-520).
    Expert modules find their engine through ``module._fsdp_run``."""

    def __init__(self, dense: FSDPEngine, expert: FSDPEngine, ep_group: Optional[dist.ProcessGroup] = None):
        self.dense, self.expert = dense, expert
        # ranks that hold DIFFERENT experts: the expert part of the global gradient norm is summed over it
        self.ep_group = ep_group
        for u in expert.units:
            u.recompute = False
            u.module._fsdp_run = expert.run
        self.device, self.rank, self.world = dense.device, dense.rank, dense.world
        self.group = dense.group

    @property
    def engines(self):
        return (self.dense, self.expert)

    def run(self, module, *a, **k):
        return self.dense.run(module, *a, **k)

    def materialize(self, init_fn):
        for e in self.engines:
            e.materialize(init_fn)

    def set_lr(self, lr):
        for e in self.engines:
            e.set_lr(lr)

    def end_micro_step(self):
        for e in self.engines:
            e.end_micro_step()

    def finish_step(self, lr=None):
        """Joint gradient clipping: the global norm combines both engines' squared norms."""
        if self.dense.opt.clip_grad > 0:
            return _joint_clip_finish(self.engines, {id(self.expert): self.ep_group})
        norms = [e.finish_step(lr) for e in self.engines]
        return norms[0]

    def named_full_params(self):
        for e in self.engines:
            yield from e.named_full_params()

    def load_full_params(self, getter):
        return sum((e.load_full_params(getter) for e in self.engines), [])

    def sharded_state(self):
        out = {}
        for tag, e in zip(("dense", "expert"), self.engines):
            out.update({f"{tag}/{k}": v for k, v in e.sharded_state().items()})
        return out

    def load_sharded_state(self, state: dict, load_optim: bool = True) -> None:
        """Inverse of ``sharded_state``: strips the ``dense/`` / ``expert/`` tag and hands each engine its records."""
        for tag, e in zip(("dense", "expert"), self.engines):
            pre = tag + "/"
            e.load_sharded_state({k[len(pre):]: v for k, v in state.items() if k.startswith(pre)}, load_optim=load_optim)

    def param_count(self):
        return sum(e.param_count() for e in self.engines)


def _joint_clip_finish(engines, extra_groups: Optional[dict] = None):
    """Deferred update of several engines under ONE clip coefficient.  The squared norm of an engine's gradients is
    summed over its own sharding group; for expert parameters it is summed once more over the expert-parallel group
    (``extra_groups[id(engine)]``), because ranks of that group hold different experts.  The total is then identical
    on every rank (reference: fsdp/optimizer/clip_grad_norm.py:69-116, expert norms reduced over ep_fsdp, then ep)."""
    extra_groups = extra_groups or {}
    total = None
    for e in engines:
        e.flush_pending()
        if e.cuda:
            torch.cuda.current_stream().wait_stream(e.comm_stream)
        groups = [g for u in e.units for g in u.groups if g.trainable and g.grad32 is not None]
        if groups:
            sq = _sq_norm([g.grad32 for g in groups]) / (e.grad_accum_steps ** 2)
        else:       # still take part in the collectives below
            sq = torch.zeros((), dtype=torch.float32, device=e.device)
        if e.world > 1:
            dist.all_reduce(sq, group=e.group)
        eg = extra_groups.get(id(e))
        if eg is not None and dist.get_world_size(eg) > 1:
            dist.all_reduce(sq, group=eg)
        total = sq if total is None else total + sq
    if total is None:
        return None
    norm = total.sqrt()
    clip = engines[0].opt.clip_grad
    scale = torch.clamp(clip / (norm + 1e-6), max=1.0)
    for e in engines:
        for u in e.units:
            for g in u.groups:
                if g.trainable and g.grad32 is not None:
                    e._adamw(g, g.grad32, scale / e.grad_accum_steps)
                    g.grad32 = None
        if e._p2p is not None:
            e._p2p.step_barrier()
        e.last_grad_norm = norm
    return norm
