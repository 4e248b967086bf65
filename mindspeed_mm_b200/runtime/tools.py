"""Profiler, memory-snapshot and watchdog helpers hooked into the training loop.

* ``Profiler``        - torch.profiler over [start_step, end_step) on selected ranks, chrome/TensorBoard traces
                        (reference: mindspeed_mm/fsdp/tools/profiler.py:32-165, tools/profiler.py:57-152).
                        NVTX ranges per FSDP unit come from ``nvtx_range`` when profiling is on.
* ``MemoryProfiler``  - ``torch.cuda.memory._record_memory_history`` between two steps and a snapshot dump
                        (fsdp/tools/memory_profiler.py:21-103).
* ``Watchdog``        - host thread that expects a heartbeat every iteration; if none arrives within the
                        timeout it logs the stalled iteration, aborts the process group and exits with code 3.
                        Nothing here touches the GPU: detection is host-side by design.
"""
from __future__ import annotations

import contextlib
import os
import threading
import time
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


class Profiler:
    def __init__(self, enable=False, ranks=(0,), start_step=10, end_step=11, save_path="./profiling", with_stack=False,
                 with_memory=False, record_shapes=False, with_cpu=True, level="level1", **_):
        rank = dist.get_rank() if dist.is_initialized() else int(os.environ.get("RANK", "0"))
        self.enabled = bool(enable) and (rank in list(ranks) or -1 in list(ranks))
        self.start_step, self.end_step, self.save_path = start_step, end_step, save_path
        self.kw = dict(with_stack=with_stack, profile_memory=with_memory, record_shapes=record_shapes)
        self.with_cpu = with_cpu
        self.prof = None
        self.rank = rank

    @classmethod
    def from_config(cls, cfg) -> "Profiler":
        sp = cfg.static_param
        return cls(enable=cfg.enable, ranks=cfg.ranks, start_step=sp.start_step, end_step=sp.end_step,
                   save_path=sp.save_path, with_stack=sp.with_stack, with_memory=sp.with_memory,
                   record_shapes=sp.record_shapes, with_cpu=sp.with_cpu, level=sp.level)

    def start(self):
        if not self.enabled:
            return
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler
        acts = [ProfilerActivity.CUDA] if torch.cuda.is_available() else []
        if self.with_cpu or not acts:
            acts.append(ProfilerActivity.CPU)
        os.makedirs(self.save_path, exist_ok=True)
        self.prof = profile(activities=acts,
                            schedule=schedule(wait=0, warmup=0, active=max(1, self.end_step - self.start_step),
                                              repeat=1, skip_first=self.start_step),
                            on_trace_ready=tensorboard_trace_handler(self.save_path, worker_name=f"rank{self.rank}"),
                            **self.kw)
        self.prof.start()

    def step(self):
        if self.prof is not None:
            self.prof.step()

    def stop(self):
        if self.prof is not None:
            self.prof.stop()
            self.prof = None


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    if enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class MemoryProfiler:
    def __init__(self, enable=False, start_step=1, end_step=2, save_path="./memory_snapshot", dump_ranks=(0,),
                 stacks="all", max_entries=None, mem_info=False, **_):
        rank = dist.get_rank() if dist.is_initialized() else int(os.environ.get("RANK", "0"))
        self.enabled = bool(enable) and rank in list(dump_ranks) and torch.cuda.is_available()
        self.start_step, self.end_step, self.save_path, self.rank = start_step, end_step, save_path, rank
        self.stacks, self.max_entries, self.mem_info = stacks, max_entries, mem_info
        self.recording = False

    def step(self, iteration: int):
        if not self.enabled:
            return
        if iteration == self.start_step and not self.recording:
            torch.cuda.memory._record_memory_history(enabled="all", stacks=self.stacks,
                                                     max_entries=self.max_entries or 100000)
            self.recording = True
        elif iteration == self.end_step and self.recording:
            os.makedirs(self.save_path, exist_ok=True)
            torch.cuda.memory._dump_snapshot(os.path.join(self.save_path, f"snapshot_rank{self.rank}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)
            self.recording = False
        if self.mem_info:
            print(f"[Rank {self.rank}] iteration {iteration} allocated {torch.cuda.memory_allocated() >> 20} MiB "
                  f"reserved {torch.cuda.memory_reserved() >> 20} MiB", flush=True)


class Watchdog:
    """``beat(iteration)`` must be called at least every ``timeout_s`` seconds once started."""

    def __init__(self, timeout_s: float, on_timeout: Optional[Callable[[int, float], None]] = None, poll_s: float = 0.5):
        self.timeout_s, self.poll_s = timeout_s, poll_s
        self.on_timeout = on_timeout or self._default
        self._last = time.monotonic()
        self._iter = -1
        self._stop = threading.Event()
        self.fired = False
        self._thread: Optional[threading.Thread] = None

    def start(self):
        if self.timeout_s and self.timeout_s > 0 and self._thread is None:
            self._last = time.monotonic()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def beat(self, iteration: int):
        self._last = time.monotonic()
        self._iter = iteration

    def stop(self):
        self._stop.set()

    def _run(self):
        while not self._stop.wait(self.poll_s):
            idle = time.monotonic() - self._last
            if idle > self.timeout_s:
                self.fired = True
                self.on_timeout(self._iter, idle)
                return

    @staticmethod
    def _default(iteration: int, idle: float):
        print(f"[watchdog] no progress for {idle:.0f}s after iteration {iteration}; aborting this rank", flush=True)
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        finally:
            os._exit(3)


class PeerHeartbeat:
    """Failure detection between ranks on the host: every rank publishes ``hb/<rank> = (iteration, wall time)`` in
    a key-value store after each step and checks its peers before the next launch.  A peer whose last beat is older
    than ``timeout_s`` (or that announced ``leave()``) is reported, so the survivors stop BEFORE issuing another
    collective instead of hanging in it.  The store is any ``torch.distributed.Store`` (TCPStore in production,
    HashStore in single-process tests)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 60.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s
        self.beat(-1)

    def beat(self, iteration: int) -> None:
        self.store.set(f"hb/{self.rank}", f"{iteration}:{time.time():.3f}")

    def leave(self, reason: str = "exit") -> None:
        """A rank that stops on purpose (between steps, with nothing in flight) says so."""
        self.store.set(f"hb/{self.rank}", f"left:{reason}")

    def failed_peers(self) -> list:
        """Ranks that left or whose heartbeat is stale."""
        now, bad = time.time(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = self.store.get(f"hb/{r}").decode()
            except Exception:  # noqa: BLE001 - key never written: the rank never joined
                bad.append((r, "never joined"))
                continue
            if v.startswith("left:"):
                bad.append((r, v[5:]))
            elif now - float(v.split(":")[1]) > self.timeout_s:
                bad.append((r, f"no heartbeat for {now - float(v.split(':')[1]):.1f}s"))
        return bad


def estimate_training_memory(n_params: float, shard_world: int = 1, tp: int = 1, param_bytes: int = 2, grad_bytes: int = 4,
                             optimizer_bytes: int = 12, activation_bytes_per_layer: float = 0.0, n_layers: int = 0,
                             recompute_layers: int = 0, layer_input_bytes: float = 0.0, largest_unit_params: float = 0.0,
                             workspace_gb: float = 2.0, reserve_gb: float = 2.0) -> dict:
    """Back-of-envelope memory model of one rank, in GiB (the reference ships the same kind of estimate as a script:
    mindspeed_mm/tools/mem_analysis.py).

    static  = sharded bf16 parameters + sharded fp32 master / Adam moments (``optimizer_bytes`` per parameter) + the
              gradient shard; ZeRO-3 additionally keeps two gathered units and one full-size gradient buffer of the
              largest unit alive (prefetch + compute).
    active  = saved activations of the layers that keep their graph + only the layer inputs of the recomputed ones.
    """
    gib = float(1 << 30)
    shard = n_params / max(tp, 1) / max(shard_world, 1)
    static = shard * (param_bytes + grad_bytes + optimizer_bytes) / gib
    gathered = largest_unit_params / max(tp, 1) * (2 * param_bytes + grad_bytes) / gib if shard_world > 1 else 0.0
    kept = max(n_layers - recompute_layers, 0)
    active = (kept * activation_bytes_per_layer + recompute_layers * layer_input_bytes) / gib
    total = static + gathered + active + workspace_gb + reserve_gb
    return dict(static_gb=static, gathered_units_gb=gathered, activation_gb=active, workspace_gb=workspace_gb,
                reserve_gb=reserve_gb, total_gb=total)
