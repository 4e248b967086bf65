"""Wan DiT under FSDP + Ulysses sequence parallelism (gloo): one optimizer step equals the single-process step."""
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


def main():
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
