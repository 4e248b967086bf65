"""Hybrid Ulysses x ring attention and chunked Ulysses (FPDT) under gloo, world 4 = ring 2 x ulysses 2."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.ops import reference as ref  # noqa: E402
from mindspeed_mm_b200.parallel.cp.hybrid import fpdt_attention, usp_attention, usp_local_indices  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    U = 2
    R = world // U
    uly_rank, ring_rank = rank % U, rank // U
    uly_groups = [dist.new_group([r * U + u for u in range(U)]) for r in range(R)]
    ring_groups = [dist.new_group([r * U + u for r in range(R)]) for u in range(U)]
    ug, rg = uly_groups[ring_rank], ring_groups[uly_rank]
    torch.manual_seed(0)
    B, S, N, NKV, D = 1, 32 * world, 4, 2, 16
    q0, k0, v0 = torch.randn(B, S, N, D), torch.randn(B, S, NKV, D), torch.randn(B, S, NKV, D)
    do0 = torch.randn(B, S, N, D)
    ok = True

    def check(tag, pairs, tol=3e-4):
        nonlocal ok
        for name, a, b in pairs:
            err = (a - b).abs().max().item()
            if err > tol:
                ok = False
                print(f"rank {rank} {tag} {name} err {err}")

    for causal in (False, True):
        qf, kf, vf = (t.clone().requires_grad_() for t in (q0, k0, v0))
        of = ref.attention_dense(qf, kf, vf, causal=causal)
        of.backward(do0)
        idx = usp_local_indices(S, R, ring_rank, U, uly_rank, causal)
        ql, kl, vl = (t[:, idx].clone().requires_grad_() for t in (q0, k0, v0))
        o = usp_attention(ql, kl, vl, ug, rg, causal=causal)
        o.backward(do0[:, idx])
        check(f"usp causal={causal}", (("out", o, of[:, idx]), ("dq", ql.grad, qf.grad[:, idx]),
                                       ("dk", kl.grad, kf.grad[:, idx]), ("dv", vl.grad, vf.grad[:, idx])))
        # FPDT over the whole world as one Ulysses group, contiguous shards, chunk = half of the local sequence
        n = S // world
        sl = slice(rank * n, (rank + 1) * n)
        ql, kl, vl = (t[:, sl].clone().requires_grad_() for t in (q0, k0, v0))
        o = fpdt_attention(ql, kl, vl, dist.group.WORLD, chunk=n // 2, causal=causal)
        o.backward(do0[:, sl])
        check(f"fpdt causal={causal}", (("out", o, of[:, sl]), ("dq", ql.grad, qf.grad[:, sl]),
                                        ("dk", kl.grad, kf.grad[:, sl]), ("dv", vl.grad, vf.grad[:, sl])))
    t = torch.tensor([int(ok)])
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_usp_check world={world} ring={R} ulysses={U} ok={bool(t.item())}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if t.item() else 1)


if __name__ == "__main__":
    main()
