"""Wan DiT under FSDP + Ulysses sequence parallelism.
default (gloo, CPU): one optimizer step equals the single-process step.
--cuda (NCCL bootstrap, >= 2 GPUs, bf16, native kernels): the fused peer-memory Ulysses path (collectives inside the
projection GEMMs, forward and backward) gives the same loss and the same reduced gradients as the all-to-all path."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.api import stable_init_fn  # noqa: E402
from mindspeed_mm_b200.models.diffusion import FlowMatchScheduler  # noqa: E402
from mindspeed_mm_b200.models.wan import SoRAModel, WanConfig, WanDiT  # noqa: E402
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig  # noqa: E402
from mindspeed_mm_b200.parallel.state import init_parallel_state, reset_parallel_state  # noqa: E402


def build(group):
    cfg = WanConfig.tiny()
    with torch.device("meta"):
        net = WanDiT(cfg)
    model = SoRAModel(net, FlowMatchScheduler(), seed=0)
    eng = FSDPEngine(model.fsdp_units(), group=group, device="cpu", param_dtype=torch.float32,
                     opt=OptimConfig(lr=1e-2, weight_decay=0.0), no_recompute=())
    eng.materialize(stable_init_fn(0.05, 0))
    return model, eng


def step(model, eng, batch):
    model.generator.manual_seed(0)
    eng.set_lr(1e-2)
    loss = model(batch, run=eng.run)
    loss.backward()
    eng.end_micro_step()
    eng.finish_step()
    return float(loss.detach())


def cuda_main():
    import mindspeed_mm_b200.models.wan as wan
    from mindspeed_mm_b200 import ops
    from mindspeed_mm_b200.ops import native
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    ops.set_tier("native")
    torch.manual_seed(0)
    cfg = WanConfig(hidden_size=256 * world // 2, ffn_dim=512, num_heads=4 * world // 2, num_layers=2, text_dim=64, text_len=16,
                    freq_dim=32)
    # `world` frames of 9 x 7 tokens: 63 tokens per rank (odd on purpose: no row-count alignment is needed)
    batch = dict(latents=torch.randn(1, 16, world, 18, 14).to(dev, torch.bfloat16),
                 prompt=torch.randn(1, 16, 64).to(dev, torch.bfloat16))
    ps = init_parallel_state(world_size=world, device_type="cuda", ulysses_parallel_size=world)
    results = {}
    for path in ("nccl", "fused"):
        wan._ULYSSES_PATH = path
        with torch.device("meta"):
            net = WanDiT(cfg)
        model = SoRAModel(net, FlowMatchScheduler(), seed=0)
        eng = FSDPEngine(model.fsdp_units(), group=ps.get_fsdp_group(), device=dev, param_dtype=torch.bfloat16,
                         opt=OptimConfig(lr=1e-3, weight_decay=0.0, clip_grad=1e9), no_recompute=())
        eng.materialize(stable_init_fn(0.05, 0))
        # the blocks' modulation / gates start at zero in a fresh model, which would hide the attention path
        for u in eng.units:
            for g_ in u.groups:
                g_.shard16.add_(0.02 * torch.randn(g_.shard16.shape, device=dev, generator=torch.Generator(dev).manual_seed(
                    1234 + eng.rank)).to(torch.bfloat16))
                g_.master.copy_(g_.shard16)
        eng.sync_after_load()
        before = native.LAUNCHES
        losses = []
        for it in range(2):
            model.generator.manual_seed(0)
            eng.set_lr(1e-3)
            loss = model(batch, run=eng.run)
            loss.backward()
            eng.end_micro_step()
            if it == 0:
                torch.cuda.synchronize()
                grads = torch.cat([g_.grad32.flatten() for u in eng.units for g_ in u.groups if g_.grad32 is not None])
            norm = eng.finish_step()
            losses.append(float(loss.detach()))
        native.check_status()
        results[path] = (losses, grads.clone(), float(norm), native.LAUNCHES - before)
    (l_a, g_a, n_a, _), (l_b, g_b, n_b, launches) = results["nccl"], results["fused"]
    rel = float((g_a - g_b).norm() / (g_a.norm() + 1e-12))
    ok = all(abs(a - b) <= 2e-2 * max(1.0, abs(a)) for a, b in zip(l_a, l_b)) and rel < 3e-2 and float(g_a.norm()) > 0
    f = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(f, op=dist.ReduceOp.MIN)
    print(f"[rank {rank}] losses nccl {l_a} fused {l_b} | reduced-gradient rel L2 diff {rel:.3e} | grad norm {n_a:.4f} vs {n_b:.4f}",
          flush=True)
    if rank == 0:
        print(f"dist_wan_check cuda world={world} ok={bool(f.item())}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if f.item() else 1)


def main():
    if "--cuda" in sys.argv:
        return cuda_main()
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    batch = dict(latents=torch.randn(1, 16, 3, 8, 8), prompt=torch.randn(1, 16, 64))
    ps = init_parallel_state(world_size=world, device_type="cpu", ulysses_parallel_size=world)
    model, eng = build(ps.get_fsdp_group())
    l_sp = step(model, eng, batch)
    got = {n: t.detach().clone() for n, t in eng.named_full_params()}
    reset_parallel_state()
    init_parallel_state(world_size=1, device_type="cpu")
    ref_model, ref_eng = build(False)
    l_ref = step(ref_model, ref_eng, batch)
    ok = abs(l_sp - l_ref) < 1e-5
    worst = 0.0
    for n, t in ref_eng.named_full_params():
        d = (got[n] - t).abs().max().item()
        worst = max(worst, d)
        if d > 2e-4:
            ok = False
            if rank == 0:
                print(f"param mismatch {n}: {d}")
    f = torch.tensor([int(ok)])
    dist.all_reduce(f, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_wan_check world={world} loss {l_sp:.6f} vs {l_ref:.6f} max_param_diff={worst:.2e} ok={bool(f.item())}")
    dist.destroy_process_group()
    sys.exit(0 if f.item() else 1)


if __name__ == "__main__":
    main()
