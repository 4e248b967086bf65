"""Dynamic data-parallel x context-parallel split on gloo world 4: group membership per split, the choice from the
longest sequence of all ranks, the batch exchange inside a context-parallel group, the ParallelState follows."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.parallel.dynamic_dpcp import DynamicDPCP  # noqa: E402
from mindspeed_mm_b200.parallel.state import init_parallel_state  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ps = init_parallel_state(world_size=world, device_type="cpu", fully_shard_parallel_size=world)
    dyn = DynamicDPCP(max_tokens_per_rank=4096, max_cp=4, parallel_state=ps)
    ok = dyn.options == [1, 2, 4]
    batch = dict(input_ids=torch.full((8,), rank), meta=[rank, "x"])
    # short sequences everywhere: one sample per rank
    out = dyn.step(batch, [1000 + rank])
    ok &= dyn.cp == 1 and len(out) == 1 and out[0] is batch
    # rank 3 meets a 6000-token sequence: two ranks per sequence
    out = dyn.step(batch, [6000] if rank == 3 else [500])
    ok &= dyn.cp == 2 and ps.size("cp") == 2 and ps.size("dp") == 2 and dyn.cp_rank == rank % 2
    first = rank - rank % 2
    ok &= [int(b["input_ids"][0]) for b in out] == [first, first + 1] and out[1]["meta"] == [first + 1, "x"]
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=dyn.cp_group)
    ok &= float(t) == float(first + first + 1)
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=dyn.dp_group)
    ok &= float(t) == float(rank % 2 + rank % 2 + 2)
    ok &= ps.group("ulysses") is dyn.cp_group
    # 15000 tokens: the whole world on one sequence
    out = dyn.step(batch, [15000] if rank == 0 else [10])
    ok &= dyn.cp == 4 and [int(b["input_ids"][0]) for b in out] == [0, 1, 2, 3] and dyn.dp_group is None
    # and back
    out = dyn.step(batch, [100])
    ok &= dyn.cp == 1 and ps.size("cp") == 1 and len(out) == 1
    try:
        dyn.choose([17000 * 4])
        ok = False
    except ValueError:
        pass
    flag = torch.tensor([float(ok)])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"ok={bool(flag.item())}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
