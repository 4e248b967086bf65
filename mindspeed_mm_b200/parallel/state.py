"""Process-group topology: one DeviceMesh for dense parallelism, one for experts.

Dense mesh dims (outer -> inner): ``pp, dp_replicate, dp_shard, ring, ulysses, tp`` with the
flattened views ``dp`` (replicate x shard), ``cp`` (ring x ulysses), ``dp_shard_cp`` (the
group FSDP shards over: a context-parallel rank holds a different slice of the same sample, so
parameters are sharded over shard x cp) and ``dp_cp``.  Expert mesh over the same ranks:
``pp, edp, efsdp, ep``.  Reference: mindspeed_mm/fsdp/distributed/parallel_state.py:31-184
(five dense dims + three expert dims); ``pp`` and ``tp`` are first-class here because the
Megatron-style backend shares this runtime instead of a second set of ``mpu`` globals.

tp is innermost so that tensor-parallel peers are neighbouring GPUs; on one NVSwitch domain all
peers are equidistant, so the order only matters across nodes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

_STATE: Optional["ParallelState"] = None

DENSE_DIMS = ("pp", "dp_replicate", "dp_shard", "ring", "ulysses", "tp")
EXPERT_DIMS = ("pp", "edp", "efsdp", "ep")


@dataclass
class ParallelSizes:
    world_size: int
    pipeline_parallel_size: int = 1
    data_parallel_replicate_size: int = 1
    fully_shard_parallel_size: int | str = "auto"
    ring_attention_size: int = 1
    ulysses_parallel_size: int = 1
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    expert_fully_shard_parallel_size: int | str = "auto"

    def resolve(self) -> "ParallelSizes":
        """Size algebra of ParallelArguments.model_post_init (fsdp/params/parallel_args.py:98-152)."""
        w = self.world_size
        # hybrid sharding: a shard size smaller than the data-parallel extent implies replica groups
        # (fsdp/distributed/parallel_state.py:109-113 builds the same 2-D mesh when sharding_size < world)
        if self.fully_shard_parallel_size not in ("auto", None, -1) and self.data_parallel_replicate_size == 1:
            rest = (self.pipeline_parallel_size * self.ring_attention_size * self.ulysses_parallel_size
                    * self.tensor_parallel_size * int(self.fully_shard_parallel_size))
            if rest and w % rest == 0 and w // rest > 1:
                self.data_parallel_replicate_size = w // rest
        fixed = (self.pipeline_parallel_size * self.data_parallel_replicate_size * self.ring_attention_size
                 * self.ulysses_parallel_size * self.tensor_parallel_size)
        if w % fixed:
            raise ValueError(f"world size {w} is not divisible by pp*replicate*ring*ulysses*tp = {fixed}")
        if self.fully_shard_parallel_size in ("auto", None, -1):
            self.fully_shard_parallel_size = w // fixed
        if fixed * self.fully_shard_parallel_size != w:
            raise ValueError(
                f"pp({self.pipeline_parallel_size}) x replicate({self.data_parallel_replicate_size}) x "
                f"shard({self.fully_shard_parallel_size}) x ring({self.ring_attention_size}) x "
                f"ulysses({self.ulysses_parallel_size}) x tp({self.tensor_parallel_size}) != world size {w}")
        per_stage = w // self.pipeline_parallel_size
        ep = self.expert_parallel_size
        if per_stage % ep:
            raise ValueError(f"expert_parallel_size {ep} must divide ranks per pipeline stage {per_stage}")
        if self.expert_fully_shard_parallel_size in ("auto", None, -1):
            self.expert_fully_shard_parallel_size = per_stage // ep // self.data_parallel_replicate_size \
                if (per_stage // ep) % self.data_parallel_replicate_size == 0 else per_stage // ep
        if (per_stage // ep) % self.expert_fully_shard_parallel_size:
            raise ValueError("expert_fully_shard_parallel_size must divide ranks_per_stage / expert_parallel_size")
        return self

    @property
    def edp(self) -> int:
        return self.world_size // self.pipeline_parallel_size // self.expert_parallel_size \
            // self.expert_fully_shard_parallel_size


class ParallelState:
    def __init__(self, sizes: ParallelSizes, device_type: str = "cpu"):
        s = sizes.resolve()
        self.sizes = s
        self.device_type = device_type
        self.world_size = s.world_size
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self._groups: Dict[str, Optional[dist.ProcessGroup]] = {}
        self._sizes: Dict[str, int] = dict(
            pp=s.pipeline_parallel_size, dp_replicate=s.data_parallel_replicate_size,
            dp_shard=s.fully_shard_parallel_size, ring=s.ring_attention_size, ulysses=s.ulysses_parallel_size,
            tp=s.tensor_parallel_size, ep=s.expert_parallel_size, efsdp=s.expert_fully_shard_parallel_size,
            edp=s.edp)
        self._sizes.update(dp=self._sizes["dp_replicate"] * self._sizes["dp_shard"],
                           cp=self._sizes["ring"] * self._sizes["ulysses"])
        self._sizes.update(dp_shard_cp=self._sizes["dp_shard"] * self._sizes["cp"],
                           dp_cp=self._sizes["dp"] * self._sizes["cp"])
        self.mesh: Optional[DeviceMesh] = None
        self.ep_mesh: Optional[DeviceMesh] = None
        if s.world_size > 1:
            if not dist.is_initialized():
                raise RuntimeError("init_process_group must be called before building a multi-rank ParallelState")
            self.mesh = init_device_mesh(device_type, tuple(self._sizes[d] for d in DENSE_DIMS),
                                         mesh_dim_names=DENSE_DIMS)
            self.ep_mesh = init_device_mesh(device_type, tuple(self._sizes[d] for d in EXPERT_DIMS),
                                            mesh_dim_names=EXPERT_DIMS)
            for d in DENSE_DIMS:
                self._groups[d] = self.mesh.get_group(d)
            for d in EXPERT_DIMS[1:]:
                self._groups[d] = self.ep_mesh.get_group(d)
            self._groups["dp"] = self._flat(self.mesh, ("dp_replicate", "dp_shard"), "dp")
            self._groups["cp"] = self._flat(self.mesh, ("ring", "ulysses"), "cp")
            self._groups["dp_shard_cp"] = self._flat(self.mesh, ("dp_shard", "ring", "ulysses"), "dp_shard_cp")
            self._groups["dp_cp"] = self._flat(self.mesh, ("dp_replicate", "dp_shard", "ring", "ulysses"), "dp_cp")
            self._groups["efsdp_ep"] = self._flat(self.ep_mesh, ("efsdp", "ep"), "efsdp_ep")

    @staticmethod
    def _flat(mesh: DeviceMesh, dims, name):
        return mesh[dims]._flatten(name).get_group()

    # generic accessors ------------------------------------------------------------------------
    def size(self, dim: str) -> int:
        return self._sizes.get(dim, 1) if dim != "efsdp_ep" else self._sizes["efsdp"] * self._sizes["ep"]

    def group(self, dim: str) -> Optional[dist.ProcessGroup]:
        return self._groups.get(dim)

    def rank_in(self, dim: str) -> int:
        g = self._groups.get(dim)
        return dist.get_rank(g) if g is not None else 0

    def enabled(self, dim: str) -> bool:
        return self.size(dim) > 1

    # named getters the model code uses (same names as the reference's generated ones) ---------
    def get_fsdp_group(self):
        return self.group("dp_shard_cp")

    def get_fsdp_world_size(self):
        return self.size("dp_shard_cp")

    def get_dp_rank(self):
        return self.rank_in("dp")

    def get_dp_world_size(self):
        return self.size("dp")

    def get_ulysses_group(self):
        return self.group("ulysses")

    def get_ring_group(self):
        return self.group("ring")

    def get_ep_group(self):
        return self.group("ep")

    def get_tp_group(self):
        return self.group("tp")

    def get_pp_group(self):
        return self.group("pp")

    def is_pipeline_first_stage(self):
        return self.rank_in("pp") == 0

    def is_pipeline_last_stage(self):
        return self.rank_in("pp") == self.size("pp") - 1

    def describe(self) -> str:
        return " ".join(f"{k}={v}" for k, v in self._sizes.items() if v > 1) or "single"


def init_parallel_state(world_size: Optional[int] = None, device_type: Optional[str] = None, **sizes) -> ParallelState:
    """Build (or rebuild) the global state.  Keyword names follow the native YAML ``parallel:`` block."""
    global _STATE
    if world_size is None:
        world_size = dist.get_world_size() if dist.is_initialized() else 1
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    known = {f for f in ParallelSizes.__dataclass_fields__}
    _STATE = ParallelState(ParallelSizes(world_size=world_size, **{k: v for k, v in sizes.items() if k in known}),
                           device_type)
    return _STATE


def get_parallel_state() -> ParallelState:
    global _STATE
    if _STATE is None:
        _STATE = ParallelState(ParallelSizes(world_size=1))
    return _STATE


def reset_parallel_state() -> None:
    global _STATE
    _STATE = None
