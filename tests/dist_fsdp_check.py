"""Multi-rank check of the sharding engine (run under torch.distributed.run; not collected by pytest).

world=N run with one pack per rank  ==  single-process run that accumulates the same N packs.
  --device cpu  : gloo, fp32, exact to 1e-5 (plumbing of gather / reduce-scatter / sharded AdamW)
  --device cuda : NCCL bootstrap; --comm p2p uses the NVLink peer-memory kernels, --comm nccl the library path;
                  both are compared with the single-process bf16 run of rank 0.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from bench import make_batches  # noqa: E402
from mindspeed_mm_b200 import ops  # noqa: E402
from mindspeed_mm_b200.api import VLMTrainerSpec, build_vlm_trainer, stable_init_fn  # noqa: E402
from mindspeed_mm_b200.data.collate import to_device  # noqa: E402
from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel  # noqa: E402
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig  # noqa: E402


def small_cfg():
    cfg = Qwen25VLConfig.tiny()
    cfg.text.num_layers = 2
    cfg.vision.depth = 2
    cfg.vision.fullatt_block_indexes = (1,)
    return cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--comm", default="auto")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--clip", type=float, default=0.0)
    ap.add_argument("--shard-size", type=int, default=0, help="hybrid sharding: ranks per shard group (replicas = world / it)")
    ap.add_argument("--offload", action="store_true", help="optimizer state in host memory")
    ap.add_argument("--keep-gathered", action="store_true", help="reshard_after_forward = False")
    ap.add_argument("--optimizer", default="adamw", help="adamw | muon")
    ap.add_argument("--lr-scaling", action="store_true", help="vision tower at 0.1 x the learning rate")
    ap.add_argument("--recompute-layers", type=int, default=-1,
                    help=">= 0: recompute only that many decoder layers, keep the graph of the rest")
    a = ap.parse_args()
    cuda = a.device == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = small_cfg()
    spec = VLMTrainerSpec(model=cfg, lr=1e-3, lr_warmup_ratio=0.0, lr_decay_style="constant", param_dtype=dtype,
                          clip_grad=a.clip, comm=a.comm, log_interval=0, weight_decay=0.01,
                          recompute=True if a.recompute_layers < 0 else a.recompute_layers,
                          shard_size=a.shard_size or None, offload_optimizer=a.offload,
                          reshard_after_forward=not a.keep_gathered, optimizer=a.optimizer,
                          lr_scaling=((r"visual\.", 0.1),) if a.lr_scaling else ())
    tr = build_vlm_trainer(spec, device=a.device)
    rank, world = dist.get_rank(), dist.get_world_size()
    packs = [make_batches(cfg, a.steps, 512, 1, 1, 224, r, pin=False) for r in range(world)]
    losses = []
    for s in range(a.steps):
        r = tr.train_step([packs[rank][s]])
        losses.append(float(r["loss"]))
    full = {n: t.detach().float().cpu().clone() for n, t in tr.engine.named_full_params()}
    if cuda:
        from mindspeed_mm_b200.ops import native
        native.check_status()

    # single-process twin on rank 0: accumulate all ranks' packs
    ok = True
    if rank == 0:
        dev = tr.device
        with torch.device("meta"):
            model = Qwen25VLModel(cfg)
        eng = FSDPEngine(model.fsdp_units(), group=False, device=dev, param_dtype=dtype,
                         opt=OptimConfig(lr=1e-3, weight_decay=0.01, clip_grad=a.clip, kind=a.optimizer,
                                         lr_scaling=((r"visual\.", 0.1),) if a.lr_scaling else ()),
                         grad_accum_steps=world)
        eng.materialize(stable_init_fn(cfg.init_std, 0))
        ref_losses = []
        for s in range(a.steps):
            eng.set_lr(1e-3)
            ls = []
            for r in range(world):
                b = to_device(packs[r][s], dev) if cuda else packs[r][s]
                loss_sum, n = model(b, run=eng.run)
                loss = loss_sum / n
                loss.backward()
                eng.end_micro_step()
                ls.append(float(loss.detach()))
            eng.finish_step()
            ref_losses.append(sum(ls) / len(ls))
        ref = {n: t.detach().float().cpu() for n, t in eng.named_full_params()}
        tol = 2e-2 if cuda else 2e-5
        for s in range(a.steps):
            if abs(losses[s] - ref_losses[s]) > tol * max(1.0, abs(ref_losses[s])):
                ok = False
                print(f"loss mismatch step {s}: {losses[s]} vs {ref_losses[s]}")
        worst = 0.0
        for n, t in ref.items():
            # fp32/gloo: element-wise.  bf16/GPU: Adam turns rounding noise of near-zero gradients into
            # +-lr steps and bf16 storage has 2^-8 relative spacing, so compare the mean deviation instead.
            d = (full[n] - t).abs().max().item() if not cuda else (full[n] - t).abs().mean().item()
            worst = max(worst, d)
            # fp32: summation order differs with the number of ranks; Adam's normalised step turns that into ~1e-5 steps
            if d > (3e-4 if cuda else (2e-5 if world <= 2 else 5e-5)):
                ok = False
                print(f"param mismatch {n}: {d}")
        if a.shard_size:
            ok = ok and tr.engine.world == a.shard_size and tr.engine.replicas == world // a.shard_size
        print(f"dist_fsdp_check world={world} shard={tr.engine.world} replicas={tr.engine.replicas} device={a.device} comm={a.comm} "
              f"p2p={getattr(tr.engine, '_p2p', None) is not None} losses={losses} ref={ref_losses} "
              f"max_param_diff={worst:.3e} ok={ok}", flush=True)
    flag = torch.tensor([int(ok)], device=tr.device)
    dist.broadcast(flag, 0)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
