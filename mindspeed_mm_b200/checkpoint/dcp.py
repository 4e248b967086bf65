"""Training checkpoints in the torch.distributed.checkpoint (DCP) layout of the reference's native trainer.

    <save>/iter_0000010/                     DCP shards (``__{rank}_0.distcp``, ``.metadata``)
    <save>/iter_0000010/extra_state/extra_state_rank_{r}.pt
    <save>/latest_checkpointed_iteration.txt "10" (or "release" for converted weights under <save>/release/)

Keys follow the reference (mindspeed_mm/fsdp/checkpoint/dcp_checkpointer.py:44-142,155-354): ``model.<name>`` holds the
parameters, ``optimizer.state.<name>.{exp_avg,exp_avg_sq,step}`` the AdamW state, every tensor a DTensor sharded along
dim 0 over the ranks.  ``<name>`` is the Hugging Face name when the model has a name map (``ops``), so a checkpoint
written by ``mm-convert ... hf_to_dcp`` or by the reference loads here and the other way round; without a map the
internal names are used.

The sharding engine keeps flat 1/N slices, not per-parameter row shards, so saving gathers one unit at a time, maps
its tensors to the external names and keeps this rank's rows; loading reads the row shards, re-assembles one layer at
a time and writes the engine's slices.  Model weights are stored from the fp32 master copy (bf16 for frozen groups).
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .sharded import TRACKER, iter_dir, read_tracker, write_tracker

EXTRA_DIR, EXTRA_FMT = "extra_state", "extra_state_rank_{}.pt"


def _rank_world():
    return (dist.get_rank(), dist.get_world_size()) if dist.is_initialized() else (0, 1)


def _rows(n: int, rank: int, world: int):
    """torch.chunk semantics of a dim-0 shard (what DTensor ``Shard(0)`` uses for uneven sizes)."""
    per = -(-n // world)
    lo = min(rank * per, n)
    return lo, min(lo + per, n)


def _wrap(full: torch.Tensor, mesh):
    """This rank's dim-0 rows of ``full`` as a DTensor on the mesh's device (a plain host tensor without a process
    group, and for scalars)."""
    if mesh is None or full.dim() == 0:
        return full.detach().cpu().clone()
    from torch.distributed.tensor import DTensor, Shard
    rank, world = _rank_world()
    lo, hi = _rows(full.shape[0], rank, world)
    return DTensor.from_local(full[lo:hi].detach().clone(), mesh, [Shard(0)], run_check=False, shape=full.shape,
                              stride=full.contiguous().stride())


def _empty_sharded(size, dtype, mesh, device):
    """Zero DTensor of global ``size`` holding only this rank's rows (the load target of one checkpoint entry)."""
    size = tuple(size)
    if mesh is None or len(size) == 0:
        return torch.zeros(size, dtype=dtype)
    from torch.distributed.tensor import DTensor, Shard
    rank, world = _rank_world()
    lo, hi = _rows(size[0], rank, world)
    local = torch.zeros((hi - lo,) + size[1:], dtype=dtype, device=device)
    stride = torch.empty(size, device="meta").stride()
    return DTensor.from_local(local, mesh, [Shard(0)], run_check=False, shape=torch.Size(size), stride=stride)


def _group_key(name: str) -> str:
    """Tensors that a name map may merge live under one layer: everything up to the first numeric path component."""
    parts = name.split(".")
    for i, p in enumerate(parts):
        if p.isdigit():
            return ".".join(parts[:i + 1])
    return ".".join(parts[:-1])


def _full_flat(engine, g, field: str) -> torch.Tensor:
    """The whole flat buffer of one group for ``field`` (shard16 / master / exp_avg / exp_avg_sq), gathered."""
    shard = getattr(g, field)
    if shard.device != engine.device:
        shard = shard.to(engine.device)
    if engine.world == 1:
        return shard
    full = torch.empty(g.padded, dtype=shard.dtype, device=engine.device)
    dist.all_gather_into_tensor(full, shard.contiguous(), group=engine.group)
    return full


def _unit_tensors(engine, u, field: str) -> Dict[str, torch.Tensor]:
    out = {}
    for g in u.groups:
        f = field if (g.trainable or field == "shard16") else None
        if f is None:
            if field != "master":
                continue
            f = "shard16"                      # frozen parameters have no master copy: store them as they are
        flat = _full_flat(engine, g, f)
        for (n, _), off, shape, numel in zip(g.named_params, g.offsets, g.shapes, g.numels):
            out[n] = flat[off:off + numel].view(shape)
    return out


class TorchDCPCheckpointer:
    """Same interface as ``checkpoint.sharded.DistributedCheckpointer``; the files are torch DCP."""

    def __init__(self, save_dir: Optional[str], load_dir: Optional[str] = None, save_async: bool = False,
                 no_save_optim: bool = False, no_save_rng: bool = False, ops: Optional[list] = None, keep_last: int = 0):
        self.save_dir, self.load_dir = save_dir, load_dir or save_dir
        self.save_async, self.no_save_optim, self.no_save_rng, self.ops = save_async, no_save_optim, no_save_rng, ops
        self._future = None
        self._async_group = None

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _check(engine):
        if hasattr(engine, "engines"):
            raise ValueError("DCP checkpoints need every rank to hold the same logical model; expert-parallel engines "
                             "keep different experts per rank: use the sharded format (save_format: sharded)")
        _, world = _rank_world()
        if world % max(engine.world * getattr(engine, "replicas", 1), 1):
            raise ValueError("DCP checkpoints are written for data-parallel sharding (FSDP / HSDP / Ulysses) only")

    def _external(self, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if not self.ops:
            return sd
        from .hf import to_hf
        return to_hf(dict(sd), self.ops)

    def _internal(self, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if not self.ops:
            return sd
        from .hf import to_internal
        return to_internal(dict(sd), self.ops)

    # ------------------------------------------------------------------ save
    def save(self, iteration: int, engine, extra_state: Optional[dict] = None) -> str:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint import FileSystemWriter
        self._check(engine)
        self.wait()
        rank, world = _rank_world()
        d = iter_dir(self.save_dir, iteration)
        os.makedirs(os.path.join(d, EXTRA_DIR), exist_ok=True)
        extra = dict(extra_state or {})
        if self.no_save_rng:
            extra.pop("torch_rng", None)
            extra.pop("cuda_rng", None)
        torch.save(extra, os.path.join(d, EXTRA_DIR, EXTRA_FMT.format(rank)))      # first, like the reference
        mesh = _mesh_for(engine)
        model_sd, opt_state = {}, {}
        for u in engine.units:
            for n, t in self._external(_unit_tensors(engine, u, "master")).items():
                model_sd[n] = _wrap(t, mesh)
            if not self.no_save_optim and u.trainable:
                avg = self._external(_unit_tensors(engine, u, "exp_avg"))
                sq = self._external(_unit_tensors(engine, u, "exp_avg_sq"))
                step = max(g.step_count for g in u.groups)
                for n in avg:
                    opt_state[n] = {"exp_avg": _wrap(avg[n], mesh), "exp_avg_sq": _wrap(sq[n], mesh),
                                    "step": torch.tensor(float(step))}
        state = {"model": model_sd}
        if opt_state:
            state["optimizer"] = {"state": opt_state}
        writer = FileSystemWriter(d, thread_count=4, single_file_per_rank=True, sync_files=False)
        if world == 1:
            dcp.save(state, storage_writer=writer, no_dist=True)
        elif self.save_async:
            if self._async_group is None:
                self._async_group = dist.new_group(backend="gloo")
            state = _to_cpu(state)
            self._future = (dcp.async_save(state, storage_writer=writer, process_group=self._async_group), iteration)
            return d
        else:
            dcp.save(state, storage_writer=writer)
            dist.barrier()
        if rank == 0:
            write_tracker(self.save_dir, iteration)
        return d

    def wait(self) -> None:
        if self._future is not None:
            fut, iteration = self._future
            fut.result()
            self._future = None
            dist.barrier()
            if _rank_world()[0] == 0:
                write_tracker(self.save_dir, iteration)

    # ------------------------------------------------------------------ load
    def load(self, engine, iteration: Optional[int] = None, load_optim: bool = True, load_rng: bool = True,
             strict: bool = True) -> Optional[dict]:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint import FileSystemReader
        self._check(engine)
        root = self.load_dir
        if not root or not os.path.isdir(root):
            return None
        release = False
        tr = os.path.join(root, TRACKER)
        if iteration is None and os.path.exists(tr):
            tag = open(tr).read().strip()
            release = tag == "release"
            iteration = None if release else int(tag)
        if iteration is None and not release:
            return None
        d = os.path.join(root, "release") if release else iter_dir(root, iteration)
        rank, world = _rank_world()
        reader = FileSystemReader(d)
        meta = reader.read_metadata().state_dict_metadata
        mesh = _mesh_for(engine)
        dev = engine.device
        want_opt = load_optim and not release
        target: Dict[str, object] = {}
        for key, m in meta.items():
            if not hasattr(m, "size"):
                continue
            if key.startswith("model.") or (want_opt and key.startswith("optimizer.state.")):
                target[key] = _empty_sharded(m.size, m.properties.dtype, mesh, dev)
        dcp.load(target, storage_reader=reader, no_dist=(world == 1))

        def full(key):
            t = target[key]
            return t.full_tensor() if hasattr(t, "full_tensor") else t

        model_keys = sorted(k[len("model."):] for k in target if k.startswith("model."))
        layers: Dict[str, List[str]] = {}
        for k in model_keys:
            layers.setdefault(_group_key(k), []).append(k)
        tables = {"master": {}, "exp_avg": {}, "exp_avg_sq": {}}
        steps = {}
        for _, names in layers.items():                      # one layer's tensors are complete on every rank at a time
            tables["master"].update(self._internal({n: full("model." + n) for n in names}))
            if want_opt and all(f"optimizer.state.{n}.exp_avg" in target for n in names):
                tables["exp_avg"].update(self._internal({n: full(f"optimizer.state.{n}.exp_avg") for n in names}))
                tables["exp_avg_sq"].update(self._internal({n: full(f"optimizer.state.{n}.exp_avg_sq") for n in names}))
        if want_opt:
            for key in target:
                if key.endswith(".step") and key.startswith("optimizer.state."):
                    steps[key] = int(float(full(key)))
        missing = _fill_engine(engine, tables, max(steps.values()) if steps else None)
        if strict and missing:
            raise KeyError(f"missing in checkpoint: {missing[:8]}{'...' if len(missing) > 8 else ''}")
        if release:
            return {}
        ex = os.path.join(d, EXTRA_DIR, EXTRA_FMT.format(rank))
        if not os.path.exists(ex):
            ex = os.path.join(d, EXTRA_DIR, EXTRA_FMT.format(0))
        extra = torch.load(ex, map_location="cpu", weights_only=False) if os.path.exists(ex) else {}
        if not load_rng:
            extra.pop("torch_rng", None)
            extra.pop("cuda_rng", None)
        return extra


def _mesh_for(engine):
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    from torch.distributed.device_mesh import init_device_mesh
    return init_device_mesh(engine.device.type, (dist.get_world_size(),))


def _to_cpu(obj):
    """Plain tensors to host memory before a background save (DTensors are staged by the DCP writer itself)."""
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, torch.Tensor) and not hasattr(obj, "to_local"):
        return obj.cpu()
    return obj


def _fill_engine(engine, tables: Dict[str, Dict[str, torch.Tensor]], step: Optional[int]) -> List[str]:
    """Write full tensors (internal names) into the engine's flat shards: bf16 shard + fp32 master from ``master``,
    the moments when present.  Returns the parameter names the checkpoint did not have."""
    missing = []
    for u in engine.units:
        for g in u.groups:
            def build(table, dtype):
                flat = torch.zeros(g.padded, dtype=dtype, device=engine.device)
                got = True
                for (n, _), off, shape, numel in zip(g.named_params, g.offsets, g.shapes, g.numels):
                    t = table.get(n)
                    if t is None:
                        got = False
                        if table is tables["master"]:
                            missing.append(n)
                        continue
                    if tuple(t.shape) != tuple(shape):
                        raise ValueError(f"shape mismatch for {n}: checkpoint {tuple(t.shape)} vs model {tuple(shape)}")
                    flat[off:off + numel].copy_(t.reshape(-1).to(engine.device, dtype))
                return g.local_slice(flat), got
            src, got = build(tables["master"], torch.float32)
            if not got and any(n in missing for n, _ in g.named_params):
                # keep what the engine already holds for parameters the checkpoint does not have
                cur = _full_flat(engine, g, "master" if g.trainable else "shard16").float()
                flat = torch.zeros(g.padded, dtype=torch.float32, device=engine.device)
                flat.copy_(cur)
                for (n, _), off, shape, numel in zip(g.named_params, g.offsets, g.shapes, g.numels):
                    t = tables["master"].get(n)
                    if t is not None:
                        flat[off:off + numel].copy_(t.reshape(-1).to(engine.device, torch.float32))
                src = g.local_slice(flat)
            g.shard16.copy_(src.to(g.shard16.dtype))
            if g.trainable:
                g.master.copy_(src.to(g.master.device))
                if tables["exp_avg"]:
                    a, ok_a = build(tables["exp_avg"], torch.float32)
                    b, ok_b = build(tables["exp_avg_sq"], torch.float32)
                    if ok_a and ok_b:
                        g.exp_avg.copy_(a.to(g.exp_avg.device))
                        g.exp_avg_sq.copy_(b.to(g.exp_avg_sq.device))
                        if step is not None:
                            g.step_count = step
    engine.sync_after_load()
    return missing
