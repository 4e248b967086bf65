"""Tensor-parallel linears under sequence parallelism on GPUs (>= 2, run with torch.distributed.run): the fused
GEMM + collective kernels (forward and backward) against the same layers on torch.distributed collectives."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.comm import fused  # noqa: E402
from mindspeed_mm_b200.ops import native  # noqa: E402
from mindspeed_mm_b200.parallel.tp import ColumnParallelLinear, RowParallelLinear  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, W = dist.get_rank(), dist.get_world_size()
    g = dist.group.WORLD
    ops.set_tier("native")
    torch.manual_seed(0)
    S_local, H, F = 256, 512, 1024 * W
    col = ColumnParallelLinear(H, F, g, bias=True, sequence_parallel=True).to(dev, torch.bfloat16)
    row = RowParallelLinear(F, H, g, bias=True, sequence_parallel=True).to(dev, torch.bfloat16)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    with torch.no_grad():
        for p in (col.weight, row.weight):
            p.copy_((0.05 * torch.randn(p.shape, device=dev, generator=gen)).to(torch.bfloat16))
        col.bias.copy_((0.1 * torch.randn(col.bias.shape, device=dev, generator=gen)).to(torch.bfloat16))
    x0 = (0.5 * torch.randn(S_local, H, device=dev, generator=gen)).to(torch.bfloat16)
    gy = torch.randn(S_local, H, device=dev, generator=gen).to(torch.bfloat16)

    def run():
        for p in list(col.parameters()) + list(row.parameters()):
            p.grad = None
        x = x0.clone().requires_grad_()
        y = row(ops.gelu_tanh(col(x)))
        y.backward(gy)
        return [y.detach().float(), x.grad.float(), col.weight.grad.float(), col.bias.grad.float(), row.weight.grad.float()]

    before = native.LAUNCHES
    got = run()
    used_fused = len(fused._SHARED) >= 2
    real = fused.fused_supported
    fused.fused_supported = lambda x: False            # same layers on torch.distributed collectives
    try:
        want = run()
    finally:
        fused.fused_supported = real
    ok = used_fused
    names = ["y", "dx", "d col.weight", "d col.bias", "d row.weight"]
    for n, a, b in zip(names, got, want):
        r = float((a - b).norm() / (b.norm() + 1e-12))
        if r > 2e-2:
            ok = False
            print(f"rank {rank} {n}: rel L2 {r}")
    native.check_status()
    f = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(f, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_tp_check world={W} fused_modules={sorted(k[0] for k in fused._SHARED)} ok={bool(f.item())}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if f.item() else 1)


if __name__ == "__main__":
    main()
