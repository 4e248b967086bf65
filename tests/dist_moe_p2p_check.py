"""Peer-memory MoE dispatcher against the NCCL all-to-all-v dispatcher (run with torch.distributed.run on >= 2 GPUs):
same outputs and the same gradients for tokens, router probabilities and expert weights."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.ops import native  # noqa: E402
from mindspeed_mm_b200.parallel import ep as epmod  # noqa: E402


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    ops.set_tier("native")
    big = "--big" in sys.argv
    T, k, E, H, F = (8192, 8, 128, 2048, 768) if big else (512, 2, 8, 256, 128)
    e_local = E // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    tokens = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev, generator=g)
    probs, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    probs = (probs / probs.sum(-1, keepdim=True)).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(7 + rank)
    gate_up = (0.05 * torch.randn(e_local, H, 2 * F, device=dev, generator=gw)).to(torch.bfloat16)
    down = (0.05 * torch.randn(e_local, F, H, device=dev, generator=gw)).to(torch.bfloat16)
    dout = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)

    def run(fn):
        t, p, a, b = (x.detach().clone().requires_grad_() for x in (tokens, probs, gate_up, down))
        out = fn(t, ids, p, a, b, E, dist.group.WORLD)
        out.backward(dout)
        return [out.detach(), t.grad, p.grad, a.grad, b.grad]

    ref = run(epmod.ep_forward_alltoall)
    got = run(epmod.ep_forward_p2p)
    ok = True
    for name, x, y in zip(("out", "dtokens", "dprobs", "dgate_up", "ddown"), got, ref):
        err = (x.float() - y.float()).abs().max().item()
        scale = y.float().abs().max().item() + 1e-6
        if err > 2e-2 * scale + 1e-3:
            ok = False
            print(f"rank {rank} {name}: err {err} scale {scale}")
    native.check_status()
    msg = ""
    if big:
        def timed(fn):
            for _ in range(3):
                run(fn)
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(5):
                run(fn)
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e) / 5], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)
        msg = f" fwd+bwd p2p {timed(epmod.ep_forward_p2p):.3f} ms vs nccl_a2a {timed(epmod.ep_forward_alltoall):.3f} ms (T={T},k={k},E={E},H={H},F={F})"
    f = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(f, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_moe_p2p_check world={world} ok={bool(f.item())}{msg}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if f.item() else 1)


if __name__ == "__main__":
    main()
