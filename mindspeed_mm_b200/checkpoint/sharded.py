"""Sharded training checkpoints: ``<save>/iter_XXXXXXX/`` + ``latest_checkpointed_iteration.txt``.

Layout and behaviour follow the reference's native checkpointer
(mindspeed_mm/fsdp/checkpoint/dcp_checkpointer.py:145-354, utils.py:21 tracker file): every rank writes
its own shard file (bf16 shards, fp32 master weights, Adam moments) and its own ``extra_state`` (iteration,
consumed samples, LR schedule, dataloader state, RNG), optionally from a background thread with at most
one save in flight (``save_async``); ``no_save_optim / no_save_rng / no_load_optim / no_load_rng`` are
honoured.  Loading with a different world size re-slices the flat buffers (every rank reads the shard
files that overlap its new slice), so a run can resume on 1, 2, 4 or 8 GPUs.
"""
from __future__ import annotations

import json
import os
import threading
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

TRACKER = "latest_checkpointed_iteration.txt"


def iter_dir(root: str, iteration: int) -> str:
    return os.path.join(root, f"iter_{iteration:07d}")


def read_tracker(root: str) -> Optional[int]:
    p = os.path.join(root, TRACKER)
    if not os.path.exists(p):
        return None
    s = open(p).read().strip()
    return None if s == "release" or not s else int(s)


def write_tracker(root: str, iteration: int) -> None:
    tmp = os.path.join(root, TRACKER + ".tmp")
    with open(tmp, "w") as f:
        f.write(str(iteration))
    os.replace(tmp, os.path.join(root, TRACKER))


def _global_rank_world(engine):
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return engine.rank, engine.world


def _sub_engines(engine):
    """(tag, engine) pairs: one for a plain sharding engine, ``dense/`` + ``expert/`` for an ``EngineMux``."""
    subs = getattr(engine, "engines", None)
    if subs is None:
        return [("", engine)]
    return list(zip(("dense/", "expert/"), subs))


class DistributedCheckpointer:
    """One shard file per global rank.  A record of a flat group carries the rank / size of the sharding group it was
    cut for (the dense engine shards over the FSDP group, an expert engine over the expert-FSDP group), so dense and
    expert records of one file may belong to groups of different sizes."""

    def __init__(self, save_dir: Optional[str], load_dir: Optional[str] = None, save_async: bool = False,
                 no_save_optim: bool = False, no_save_rng: bool = False, keep_last: int = 0,
                 async_wait_s: float = 600.0):
        self.save_dir, self.load_dir = save_dir, load_dir or save_dir
        self.save_async, self.no_save_optim, self.no_save_rng, self.keep_last = \
            save_async, no_save_optim, no_save_rng, keep_last
        self.async_wait_s = async_wait_s
        self._inflight: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None

    # ------------------------------------------------------------------ save
    def save(self, iteration: int, engine, extra_state: Optional[dict] = None) -> str:
        self.wait()
        rank, world = _global_rank_world(engine)
        d = iter_dir(self.save_dir, iteration)
        os.makedirs(d, exist_ok=True)
        state = {}
        for key, s in engine.sharded_state().items():
            rec = dict(shard16=s["shard16"].detach().cpu().clone(), step=s["step"], numel=s["numel"],
                       world=s["world"], rank=s.get("rank", 0))
            if s["master"] is not None:
                rec["master"] = s["master"].detach().cpu().clone()
                if not self.no_save_optim:
                    rec["exp_avg"] = s["exp_avg"].detach().cpu().clone()
                    rec["exp_avg_sq"] = s["exp_avg_sq"].detach().cpu().clone()
            state[key] = rec
        extra = dict(extra_state or {})
        if self.no_save_rng:
            extra.pop("torch_rng", None)
            extra.pop("cuda_rng", None)
        shard_name = f"shard_{rank:05d}_of_{world:05d}.pt"

        def atomic_save(obj, path):
            torch.save(obj, path + ".tmp")
            os.replace(path + ".tmp", path)          # a file that exists is complete

        def write():
            try:
                atomic_save(extra, os.path.join(d, f"extra_state_{rank:05d}.pt"))
                if rank == 0:
                    with open(os.path.join(d, "meta.json"), "w") as f:
                        json.dump({"iteration": iteration, "world_size": world,
                                   "groups": {k: v["numel"] for k, v in state.items()}}, f)
                atomic_save(state, os.path.join(d, shard_name))      # last: its presence means "this rank is done"
            except BaseException as e:  # noqa: BLE001
                self._error = e

        def all_written() -> bool:
            import time
            t0 = time.time()
            want = [os.path.join(d, f"shard_{r:05d}_of_{world:05d}.pt") for r in range(world)]
            while time.time() - t0 < self.async_wait_s:
                if all(os.path.exists(w) for w in want):
                    return True
                time.sleep(0.05)
            return False

        def finish():
            write()
            # every rank must have written before the tracker moves: a collective barrier on the caller's thread for a
            # synchronous save; a background save must not issue collectives, so rank 0 watches for the files instead
            if world > 1:
                if not self.save_async:
                    dist.barrier()
                elif rank == 0 and not all_written():
                    self._error = self._error or TimeoutError(f"not every rank wrote its shard of {d}")
            if rank == 0 and self._error is None:
                write_tracker(self.save_dir, iteration)
                self._prune()

        if self.save_async:
            self._inflight = threading.Thread(target=finish, daemon=True)
            self._inflight.start()
        else:
            finish()
            if self._error:
                raise self._error
        return d

    def wait(self) -> None:
        if self._inflight is not None:
            self._inflight.join()
            self._inflight = None
        if self._error:
            e, self._error = self._error, None
            raise e

    def _prune(self):
        if self.keep_last <= 0:
            return
        its = sorted(int(n[5:]) for n in os.listdir(self.save_dir) if n.startswith("iter_"))
        import shutil
        for it in its[:-self.keep_last]:
            shutil.rmtree(iter_dir(self.save_dir, it), ignore_errors=True)

    # ------------------------------------------------------------------ load
    def load(self, engine, iteration: Optional[int] = None, load_optim: bool = True, load_rng: bool = True,
             strict: bool = True) -> Optional[dict]:
        root = self.load_dir
        if not root or not os.path.isdir(root):
            return None
        if iteration is None:
            iteration = read_tracker(root)
        if iteration is None:
            return None
        d = iter_dir(root, iteration)
        files = sorted(f for f in os.listdir(d) if f.startswith("shard_") and f.endswith(".pt"))
        if not files:
            raise FileNotFoundError(f"no shard files in {d}")
        rank, world = _global_rank_world(engine)
        old_world = int(files[0].split("_of_")[1].split(".")[0])
        if old_world == world:
            st = torch.load(os.path.join(d, files[rank]), map_location="cpu", weights_only=False)
            engine.load_sharded_state(st, load_optim=load_optim)
        else:
            self._load_resharded(engine, d, files, load_optim)
        ex = os.path.join(d, f"extra_state_{rank:05d}.pt")
        if not os.path.exists(ex):
            ex = os.path.join(d, "extra_state_00000.pt")
        extra = torch.load(ex, map_location="cpu", weights_only=False) if os.path.exists(ex) else {}
        if not load_rng:
            extra.pop("torch_rng", None)
            extra.pop("cuda_rng", None)
        return extra

    @staticmethod
    def _load_resharded(engine, d: str, files: List[str], load_optim: bool) -> None:
        """The job has a different number of ranks than the one that saved.  A group that was sharded over ALL ranks
        (then and now) is rebuilt by concatenating the old slices in rank order and cutting this rank's new slice.
        Groups sharded over a sub-group (experts under expert parallelism, tensor / pipeline parallel shards) hold
        different parameters on different ranks, so they cannot be re-cut: that is refused."""
        olds = [torch.load(os.path.join(d, f), map_location="cpu", weights_only=False) for f in files]
        _, world = _global_rank_world(engine)
        for tag, e in _sub_engines(engine):
            if e.world != world:
                raise ValueError(f"checkpoint was written by {len(files)} ranks and the '{tag or 'model'}' parameters are "
                                 f"sharded over a sub-group of {e.world}: reload with the original layout, or convert "
                                 f"through the full (HF) format")
            st = {}
            for u in e.units:
                for gi, g in enumerate(u.groups):
                    key = f"{tag}{u.name}#{gi}"
                    if any(o[key].get("world", len(files)) != len(files) for o in olds):
                        raise ValueError(f"{key} was not sharded over all {len(files)} ranks of the saving job")

                    def rebuild(field, g=g, key=key):
                        flat = torch.cat([o[key][field] for o in olds])[:g.numel]
                        out = torch.zeros(g.padded, dtype=flat.dtype)
                        out[:g.numel] = flat
                        return out[g.rank * g.shard_numel:(g.rank + 1) * g.shard_numel]

                    first = olds[0][key]
                    rec = dict(shard16=rebuild("shard16"), world=e.world, rank=e.rank, step=first["step"], master=None,
                               exp_avg=None, exp_avg_sq=None)
                    if g.trainable:
                        rec["master"] = rebuild("master" if "master" in first else "shard16")
                        if load_optim and "exp_avg" in first:
                            rec["exp_avg"], rec["exp_avg_sq"] = rebuild("exp_avg"), rebuild("exp_avg_sq")
                    st[f"{u.name}#{gi}"] = rec
            e.load_sharded_state(st, load_optim=load_optim)
