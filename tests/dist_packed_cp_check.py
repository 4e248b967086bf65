"""Packed-sequence context parallelism (all-gathered keys / values) on gloo: outputs and gradients of the local chunks
equal the single-process varlen attention on the whole packed stream."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.parallel.cp.packed import chunk_plan, packed_attention  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    lens = [5, 37, 2, 60, 16] if world == 2 else [5, 37, 2, 61, 15, 48]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T, Nq, Nkv, D = cu[-1], 4, 2, 16
    assert T % world == 0
    q = torch.randn(T, Nq, D, dtype=torch.double, requires_grad=True)
    k = torch.randn(T, Nkv, D, dtype=torch.double, requires_grad=True)
    v = torch.randn(T, Nkv, D, dtype=torch.double, requires_grad=True)
    cut = torch.tensor(cu, dtype=torch.int32)
    ref = ops.attention_varlen(q, k, v, cut, cut, max(lens), max(lens), causal=True)
    w = torch.randn_like(ref)
    (ref * w).sum().backward()
    per = T // world
    sl = slice(rank * per, (rank + 1) * per)
    ql, kl, vl = (t.detach()[sl].clone().requires_grad_() for t in (q, k, v))
    out = packed_attention(ql, kl, vl, cu, dist.group.WORLD, causal=True)
    (out * w[sl]).sum().backward()
    # the CPU reference computes in fp32 whatever the input type
    ok = torch.allclose(out, ref[sl], atol=1e-5)
    for got, full in ((ql.grad, q.grad), (kl.grad, k.grad), (vl.grad, v.grad)):
        ok &= torch.allclose(got, full[sl], atol=1e-5)
    if not ok:
        print(rank, "out", float((out - ref[sl]).abs().max()), [float((g - f[sl]).abs().max()) for g, f in
                                                                 ((ql.grad, q.grad), (kl.grad, k.grad), (vl.grad, v.grad))])
    # a chunk that starts inside a document sees that document's earlier keys
    ks, hi, cq, ck = chunk_plan(cu, world, rank)
    ok &= hi == (rank + 1) * per and cq[-1] == per and ck[-1] == hi - ks and ks <= rank * per
    flag = torch.tensor([float(ok)])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"world={world} tokens={T} ok={bool(flag.item())}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
