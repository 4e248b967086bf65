"""Context-parallel attention under gloo (run with torch.distributed.run; not collected by pytest):
Ulysses and ring (non-causal and zig-zag causal) outputs and input gradients equal single-rank attention."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.ops import reference as ref  # noqa: E402
from mindspeed_mm_b200.parallel.cp.ring import ring_attention  # noqa: E402
from mindspeed_mm_b200.parallel.cp.split import (gather_forward_split_backward, split_forward_gather_backward,  # noqa: E402
                                                  zigzag_indices)
from mindspeed_mm_b200.parallel.cp.ulysses import ulysses_attention  # noqa: E402


def main():
    cuda = "--cuda" in sys.argv
    if cuda:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = dist.group.WORLD
    torch.manual_seed(0)
    # GPU run: head dim 128 and bf16 so that the tcgen05 block kernels and the peer-memory ring transport are used
    B, S, N, NKV, D = (1, 512 * world, 4, 2, 128) if cuda else (2, 8 * world, 4, 2, 16)
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dt = torch.bfloat16 if cuda else torch.float32
    tol = 3e-2 if cuda else 2e-4
    q0, k0, v0 = (torch.randn(B, S, n, D).to(dt).to(dev) for n in (N, NKV, NKV))
    do0 = torch.randn(B, S, N, D).to(dt).to(dev)
    ok = True
    for causal in (False, True):
        qf, kf, vf = (t.clone().requires_grad_() for t in (q0, k0, v0))
        of = ref.attention_dense(qf.float(), kf.float(), vf.float(), causal=causal)
        of.backward(do0.float())
        # ---- ring (zig-zag order when causal)
        idx = (zigzag_indices(S, world, rank) if causal else torch.arange(rank * S // world, (rank + 1) * S // world)).to(dev)
        ql, kl, vl = (t[:, idx].clone().requires_grad_() for t in (q0, k0, v0))
        o = ring_attention(ql, kl, vl, g, causal=causal)
        o.backward(do0[:, idx])
        for name, a, b in (("out", o, of[:, idx]), ("dq", ql.grad, qf.grad[:, idx]), ("dk", kl.grad, kf.grad[:, idx]),
                           ("dv", vl.grad, vf.grad[:, idx])):
            err = (a.float() - b.float()).abs().max().item()
            if err > tol * max(1.0, b.float().abs().max().item()):
                ok = False
                print(f"rank {rank} ring causal={causal} {name} err {err} ref_max {b.float().abs().max().item()}", flush=True)
        # ---- ulysses (contiguous split), including split/gather autograd helpers
        if not causal:
            qu, ku, vu = (t.clone().requires_grad_() for t in (q0, k0, v0))
            qs = split_forward_gather_backward(qu, g, dim=1)
            ks = split_forward_gather_backward(ku, g, dim=1)
            vs = split_forward_gather_backward(vu, g, dim=1)
            ou = ulysses_attention(lambda a, b, c: (ops.attention_dense if cuda else ref.attention_dense)(a, b, c), qs, ks, vs, g)
            full = gather_forward_split_backward(ou, g, dim=1)
            full.backward(do0)
            for name, a, b in (("out", full, of), ("dq", qu.grad, qf.grad), ("dk", ku.grad, kf.grad), ("dv", vu.grad, vf.grad)):
                err = (a.float() - b.float()).abs().max().item()
                if err > tol * max(1.0, b.float().abs().max().item()):
                    ok = False
                    print(f"rank {rank} ulysses {name} err {err} ref_max {b.float().abs().max().item()}", flush=True)
    t = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if cuda:
        from mindspeed_mm_b200.ops import native
        native.check_status()
    if rank == 0:
        print(f"dist_cp_check world={world} device={dev.type} ok={bool(t.item())}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if t.item() else 1)


if __name__ == "__main__":
    main()
