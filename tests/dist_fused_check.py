"""Fused GEMM + collective kernels against GEMM followed by the NCCL collective (>= 2 GPUs; run with
torch.distributed.run).  Also times both with CUDA events (max over ranks)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.comm.fused import (AllGatherLinear, RowParallelLinearRS, UlyssesOutProjection,  # noqa: E402
                                           UlyssesQKVProjection)
from mindspeed_mm_b200.ops import native  # noqa: E402


def timed(fn, iters=5):
    for _ in range(2):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, W = dist.get_rank(), dist.get_world_size()
    g = dist.group.WORLD
    ok = True
    torch.manual_seed(0)
    big = "--big" in sys.argv
    # ---------------- Ulysses QKV: x_local [S_local, H] -> q|k|v of my heads over the full sequence
    H = 5120 if big else 1024
    S_local = (75600 // 8 // 128 * 128) if big else 512
    xs = torch.randn(W, S_local, H, device="cuda", dtype=torch.bfloat16) * 0.5
    w = (torch.randn(3 * H, H, device="cuda") * 0.03).to(torch.bfloat16)
    b = torch.randn(3 * H, device="cuda", dtype=torch.bfloat16)
    x = xs[rank].clone().requires_grad_()
    wq = w.clone().requires_grad_()
    proj = UlyssesQKVProjection(g, "cuda", S_local, 3 * H)
    y = proj(x, wq, b)
    # unfused reference: local GEMM, then all-to-all of head blocks
    def unfused(xl, wl):
        yl = native.gemm_nt(xl, wl, b)                                   # [S_local, 3H]
        blk = H // W
        send = yl.view(S_local, 3, W, blk).permute(2, 0, 1, 3).contiguous()    # [dst, S_local, 3, blk]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=g)                      # [src, S_local, 3, blk]
        return recv.reshape(W * S_local, 3 * blk)
    ref = unfused(xs[rank], w)
    err = (y.float() - ref.float()).abs().max().item()
    if err > 1e-2:
        ok = False
        print(f"rank {rank} ulysses fwd err {err}")
    gy = torch.randn_like(y)
    y.backward(gy)
    # reference gradients through autograd of the unfused torch path
    xr = xs[rank].clone().float().requires_grad_()
    wr = w.clone().float().requires_grad_()
    yl = torch.nn.functional.linear(xr, wr, b.float())
    blk = H // W
    send = yl.view(S_local, 3, W, blk).permute(2, 0, 1, 3).contiguous()
    gsend = torch.empty_like(send)
    dist.all_to_all_single(gsend, gy.float().view(W, S_local, 3, blk).contiguous(), group=g)
    send.backward(gsend)
    for name, a_, b_ in (("dx", x.grad, xr.grad), ("dw", wq.grad, wr.grad)):
        e_ = (a_.float() - b_).abs().max().item() / (b_.abs().max().item() + 1e-6)
        if e_ > 3e-2:
            ok = False
            print(f"rank {rank} ulysses {name} rel err {e_}")
    t_f = timed(lambda: proj(xs[rank], w, b))
    t_u = timed(lambda: unfused(xs[rank], w))
    # ---------------- row-parallel linear + reduce-scatter
    M, N, K = (8192, 8192, 29568 // 4 // 64 * 64) if big else (1024, 512, 768)
    xa = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * 0.5
    wa = (torch.randn(N, K, device="cuda") * 0.03).to(torch.bfloat16)
    rs = RowParallelLinearRS(g, "cuda", M, N)
    yo = rs(xa, wa)
    part = native.gemm_nt(xa, wa).float()
    refo = torch.empty(M // W, N, device="cuda")
    dist.reduce_scatter_tensor(refo, part, group=g)
    e2 = (yo.float() - refo).abs().max().item() / (refo.abs().max().item() + 1e-6)
    if e2 > 2e-2:
        ok = False
        print(f"rank {rank} rs fwd rel err {e2}")
    def unfused_rs():
        p_ = native.gemm_nt(xa, wa)
        o_ = torch.empty(M // W, N, device="cuda", dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(o_, p_, group=g)
        return o_
    t_rf = timed(lambda: rs(xa, wa))
    t_ru = timed(unfused_rs)
    # ---------------- sequence-parallel all-gather -> column-parallel GEMM
    Sl, Hh, Nn = (1024, 8192, 29568 // 4 // 64 * 64 * 2) if big else (256, 512, 768)
    xl = torch.randn(W, Sl, Hh, device="cuda", dtype=torch.bfloat16) * 0.5
    wc = (torch.randn(Nn, Hh, device="cuda") * 0.03).to(torch.bfloat16)
    agl = AllGatherLinear(g, "cuda", Sl, Hh)
    for rep in range(2):                                  # second call exercises the epoch counters
        ya = agl(xl[rank], wc)
    refa = native.gemm_nt(xl.reshape(W * Sl, Hh), wc)
    e3 = (ya.float() - refa.float()).abs().max().item() / (refa.float().abs().max().item() + 1e-6)
    if e3 > 1e-2:
        ok = False
        print(f"rank {rank} allgather-linear rel err {e3}")
    def unfused_ag():
        full = torch.empty(W * Sl, Hh, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, xl[rank], group=g)
        return native.gemm_nt(full, wc)
    t_af = timed(lambda: agl(xl[rank], wc))
    t_au = timed(unfused_ag)
    # ---------------- Ulysses output projection (heads come back from peers)
    So, Ho = (S_local, H) if big else (256, 1024)
    o_full = torch.randn(W * So, Ho, device="cuda", dtype=torch.bfloat16) * 0.5     # same on every rank (seeded)
    wo = (torch.randn(Ho, Ho, device="cuda") * 0.03).to(torch.bfloat16)
    cols = Ho // W
    mine = o_full[:, rank * cols:(rank + 1) * cols].contiguous()                   # my heads, all tokens
    uo = UlyssesOutProjection(g, "cuda", So, Ho)
    for rep in range(2):
        yu = uo(mine, wo)
    refu = native.gemm_nt(o_full[rank * So:(rank + 1) * So].contiguous(), wo)
    e4 = (yu.float() - refu.float()).abs().max().item() / (refu.float().abs().max().item() + 1e-6)
    if e4 > 1e-2:
        ok = False
        print(f"rank {rank} ulysses-out rel err {e4}")
    def unfused_uo():
        send = mine.view(W, So, cols).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=g)
        return native.gemm_nt(recv.permute(1, 0, 2).reshape(So, Ho), wo)
    t_of = timed(lambda: uo(mine, wo))
    t_ou = timed(unfused_uo)
    # ---------------- backward passes of the three layers above against fp32 autograd through NCCL collectives
    def rel(a_, b_):
        return (a_.float() - b_.float()).norm().item() / (b_.float().norm().item() + 1e-12)

    # row-parallel + reduce-scatter: y_l = RS(x W^T);  backward gathers the rows of g inside dx = gather(g) W
    xg, wg = xa.clone().requires_grad_(), wa.clone().requires_grad_()
    yo = rs(xg, wg)
    gy = torch.randn_like(yo)
    yo.backward(gy)
    gfull = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    dist.all_gather_into_tensor(gfull, gy, group=g)
    for name, a_, b_ in (("dx", xg.grad, gfull.float() @ wa.float()), ("dw", wg.grad, gfull.float().t() @ xa.float())):
        if rel(a_, b_) > 2e-2:
            ok = False
            print(f"rank {rank} rowparallel_rs {name} rel err {rel(a_, b_)}")
    # all-gather + column-parallel: backward pushes dA = g W as row blocks to the row owners
    xg, wg = xl[rank].clone().requires_grad_(), wc.clone().requires_grad_()
    ya = agl(xg, wg)
    gy = torch.randn_like(ya)
    ya.backward(gy)
    dA = gy.float() @ wc.float()
    dxr = torch.empty(Sl, Hh, device="cuda")
    dist.reduce_scatter_tensor(dxr, dA, group=g)
    for name, a_, b_ in (("dx", xg.grad, dxr), ("dw", wg.grad, gy.float().t() @ xl.reshape(W * Sl, Hh).float())):
        if rel(a_, b_) > 2e-2:
            ok = False
            print(f"rank {rank} allgather_linear {name} rel err {rel(a_, b_)}")
    # Ulysses output projection: backward stores the head blocks of dA = g W into the head owners
    og, wg = mine.clone().requires_grad_(), wo.clone().requires_grad_()
    yu = uo(og, wg)
    gy = torch.randn_like(yu)
    yu.backward(gy)
    dA = (gy.float() @ wo.float()).view(So, W, cols).permute(1, 0, 2).contiguous()     # [head owner, my rows, cols]
    back = torch.empty_like(dA)
    dist.all_to_all_single(back, dA, group=g)                                          # [row owner, its rows, cols]
    a_full = o_full[rank * So:(rank + 1) * So].float()
    for name, a_, b_ in (("do", og.grad, back.reshape(W * So, cols)), ("dw", wg.grad, gy.float().t() @ a_full)):
        if rel(a_, b_) > 2e-2:
            ok = False
            print(f"rank {rank} ulysses_out {name} rel err {rel(a_, b_)}")
    # Ulysses QKV with the row statistics side output, ragged rows per rank (not a multiple of 128)
    Sr = 201
    xr_ = torch.randn(W, Sr, H, device="cuda", dtype=torch.bfloat16) * 0.5
    pr = UlyssesQKVProjection(g, "cuda", Sr, 3 * H, 3, True)
    yr_, st_ = pr(xr_[rank].clone(), w, b)
    full_y = torch.nn.functional.linear(xr_.reshape(W * Sr, H).float(), w.float(), b.float()).to(torch.bfloat16).float()
    blk_ = H // W
    want = full_y.view(W * Sr, 3, W, blk_)[:, :, rank].reshape(W * Sr, 3 * blk_)
    want_ss = full_y.view(W * Sr, 3, H).pow(2).sum(-1)
    if rel(yr_, want) > 1e-2 or rel(st_, want_ss) > 1e-2:
        ok = False
        print(f"rank {rank} ulysses qkv+stats rel err {rel(yr_, want)} stats {rel(st_, want_ss)}")
    native.check_status()
    flag = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_fused_check world={W} ok={bool(flag.item())} ulysses_qkv fused {t_f:.3f} ms vs gemm+nccl_a2a {t_u:.3f} ms | "
              f"rowparallel_rs fused {t_rf:.3f} ms vs gemm+nccl_rs {t_ru:.3f} ms | allgather_linear fused {t_af:.3f} ms vs "
              f"nccl_ag+gemm {t_au:.3f} ms | ulysses_out fused {t_of:.3f} ms vs nccl_a2a+gemm {t_ou:.3f} ms "
              f"(S_local={S_local}, H={H}; M={M},N={N},K={K})",
              flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
