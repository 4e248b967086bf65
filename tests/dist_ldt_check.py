"""U-shaped edge/cloud pipeline on gloo: loss and gradients must equal the single-process model."""
import argparse
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.parallel.ldt import DisaggregatedPipeline, StageSpec, simulate_1f1b, u_shaped  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--wide", action="store_true", help="cloud stage replicated over two ranks (TP-style fan-out)")
    a = ap.parse_args()
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    fwd = dist.new_group(list(range(world)))
    bwd = dist.new_group(list(range(world)))
    torch.manual_seed(0)
    H, n_micro = 16, 4
    stages = u_shaped(0, [[1, 2]]) if a.wide else u_shaped(0, [[r] for r in range(1, world)])
    n = len(stages)
    layers = nn.ModuleList(nn.Sequential(nn.Linear(H, H), nn.Tanh()) for _ in range(n))     # same init on all ranks
    mbs = [dict(x=torch.randn(3, H), y=torch.randn(3, H)) for _ in range(n_micro)]

    def stage_fn(s, x, mb):
        h = layers[s](mb["x"] if s == 0 else x)          # raw inputs only on the edge (first stage)
        if s == n - 1:
            return ((h - mb["y"]) ** 2).mean() / n_micro  # labels only on the edge (last stage)
        return h

    pipe = DisaggregatedPipeline(stages, stage_fn, lambda s, mb: (3, H), torch.float32, "cpu", fwd, bwd)
    losses = pipe.run(mbs)
    # single-process reference
    ref = nn.ModuleList(nn.Sequential(nn.Linear(H, H), nn.Tanh()) for _ in range(n))
    ref.load_state_dict(layers.state_dict())
    total = 0.0
    for mb in mbs:
        h = mb["x"]
        for l in ref:
            h = l(h)
        loss = ((h - mb["y"]) ** 2).mean() / n_micro
        loss.backward()
        total += loss.item()
    ok = True
    for s in pipe.mine:
        for p, q in zip(layers[s].parameters(), ref[s].parameters()):
            ok &= torch.allclose(p.grad, q.grad, atol=1e-6)
    if rank == 0:
        ok &= abs(sum(l.item() for l in losses) - total) < 1e-6 and pipe.mine == [0, n - 1]
    else:
        ok &= all(p.grad is None for s in range(n) if s not in pipe.mine for p in layers[s].parameters())
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        plan = simulate_1f1b(n, n_micro, [s.ranks for s in stages])
        print(f"dist_ldt_check world={world} stages={[s.ranks for s in stages]} ops_rank0={len(plan[0])} ok={bool(flag.item())}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
