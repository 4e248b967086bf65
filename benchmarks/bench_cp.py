"""Context-parallel attention on N GPUs: ring (peer-memory transport), Ulysses (all-to-all) and packed-sequence
(all-gathered keys / values) attention, forward + backward, against the same attention on one GPU's share of the work.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29571 \
        benchmarks/bench_cp.py [--seq-per-rank 16384] [--heads 16] [--out FILE]

Timing: CUDA events on the launching stream, 2 warm-ups, 5 timed iterations, barrier + synchronize on both sides, max over
ranks.  ``ideal_ms`` = the attention FLOPs of one rank (1 / N of the whole) run as a single local call: what a transport
that costs nothing would give.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.parallel.cp.packed import packed_attention  # noqa: E402
from mindspeed_mm_b200.parallel.cp.ring import ring_attention  # noqa: E402
from mindspeed_mm_b200.parallel.cp.ulysses import ulysses_attention  # noqa: E402


def timed(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-per-rank", type=int, default=16384)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    g = dist.group.WORLD
    S, N, D = a.seq_per_rank, a.heads, 128
    torch.manual_seed(rank)
    mk = lambda *shape: torch.randn(*shape, device="cuda", dtype=torch.bfloat16).requires_grad_()
    rows = []

    def fb(fn, *ins):
        o = fn(*ins)
        o.backward(torch.ones_like(o))

    for causal in (False, True):
        q, k, v = mk(1, S, N, D), mk(1, S, N, D), mk(1, S, N, D)
        t_ring = timed(lambda: fb(lambda a_, b_, c_: ring_attention(a_, b_, c_, g, causal=causal), q, k, v))
        # one rank's share of the FLOPs as a single local call: S queries against S * world keys (half of them when causal)
        keys = S * world // (2 if causal else 1)
        kk, vv = mk(1, keys, N, D), mk(1, keys, N, D)
        t_ideal = timed(lambda: fb(lambda a_, b_, c_: ops.attention_dense(a_, b_, c_), q, kk, vv))
        rows.append(dict(op="ring_attention", causal=causal, world=world, seq_per_rank=S, heads=N, fwd_bwd_ms=round(t_ring, 3),
                         ideal_ms=round(t_ideal, 3), efficiency=round(t_ideal / t_ring, 3)))
        if not causal and N % world == 0:
            t_uly = timed(lambda: fb(lambda a_, b_, c_: ulysses_attention(lambda x, y, z: ops.attention_dense(x, y, z), a_, b_, c_, g),
                                     q, k, v))
            # Ulysses: every rank runs N / world heads over the whole sequence = the same FLOPs
            rows.append(dict(op="ulysses_attention", causal=False, world=world, seq_per_rank=S, heads=N,
                             fwd_bwd_ms=round(t_uly, 3), ideal_ms=round(t_ideal, 3), efficiency=round(t_ideal / t_uly, 3)))
    # packed stream: documents of 4096 tokens over the whole stream, GQA 16 / 4 heads
    T = S * world
    cu = list(range(0, T + 1, 4096))
    qp, kp, vp = mk(S, N, D), mk(S, max(1, N // 4), D), mk(S, max(1, N // 4), D)
    t_packed = timed(lambda: fb(lambda a_, b_, c_: packed_attention(a_, b_, c_, cu, g, causal=True), qp, kp, vp))
    cul = torch.tensor(list(range(0, S + 1, 4096)), dtype=torch.int32, device="cuda")
    t_local = timed(lambda: fb(lambda a_, b_, c_: ops.attention_varlen(a_, b_, c_, cul, cul, 4096, 4096, causal=True), qp, kp, vp))
    rows.append(dict(op="packed_cp_attention", causal=True, world=world, seq_per_rank=S, heads=N, doc_len=4096,
                     fwd_bwd_ms=round(t_packed, 3), ideal_ms=round(t_local, 3), efficiency=round(t_local / t_packed, 3)))
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if a.out:
            with open(a.out, "a") as f:
                for r in rows:
                    f.write(json.dumps(r) + "\n")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
