"""Flagship benchmark: Qwen2.5-VL-7B full-parameter finetune step, ZeRO-3 (FSDP2 semantics), bf16.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Per GPU: one packed micro-batch of 8192 tokens (4 samples x 2048 tokens, each with two 448x448 images =
2 x 256 visual tokens), activation checkpointing per layer, AdamW (lr 1e-5, wd 0, no clipping: the
reference's FSDP2 recipe, examples/qwen2.5vl/finetune_qwen2_5_vl_72b_fsdp.sh), synthetic data,
random-init weights.  Weak scaling: the global batch is N packs.

Two timed regions of K steps each, both bracketed by barrier + synchronize and timed with CUDA events
(max over ranks):
  * ``value``  - inputs already on the device (kernel-only number)
  * ``e2e``    - every step copies its inputs from pinned host memory and reads the loss back to the host,
                 through the public ``TrainEngine.train_step`` API.
Weights + optimizer state (> 100 GB) are far larger than L2, so no explicit L2 flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_CARD = 11042.0  # Qwen2.5-VL-7B finetune, mcore TP=1, tokens/s per 910B2 card (published)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of this rank's GPU through NVML (read-only) every 200 ms."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:  # noqa: BLE001
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = fn(self.h)
                for bit, nm in names.items():
                    if mask & bit:
                        self.reasons.add(nm)
            except Exception:  # noqa: BLE001
                pass
            self._stop_evt.wait(0.2)

    def stop(self):
        self._stop_evt.set()
        if self.ok:
            self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def run_reference(args):
    """The reference arm: the unmodified reference from baseline/_ref through its own native trainer
    (``baseline/reference_arm.py``).  Nothing of this repository's package is imported on this path."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm
    return reference_arm.run(args, ClockSampler)


def make_batches(cfg, n_batches, seq_len, samples_per_pack, images_per_sample, image_size, rank, pin):
    from mindspeed_mm_b200.data.collate import PackedVLMCollator
    from mindspeed_mm_b200.data.synthetic import SyntheticVLMDataset, SyntheticVLMSpec
    per = seq_len // samples_per_pack
    ds = SyntheticVLMDataset(SyntheticVLMSpec(
        seq_len=per, images_per_sample=images_per_sample, image_size=image_size, vocab_size=cfg.text.vocab_size,
        image_token_id=cfg.image_token_id, vision_start_token_id=cfg.vision_start_token_id, seed=1234 + rank,
        pixel_dtype=torch.bfloat16, patch=cfg.vision.patch_size, merge=cfg.vision.spatial_merge_size))
    col = PackedVLMCollator.for_config(cfg, pixel_dtype=torch.bfloat16, pin=pin)
    return [col([ds[b * samples_per_pack + i] for i in range(samples_per_pack)]) for b in range(n_batches)]


def run_wan(args, steps=None, nested=False):
    """Second headline workload: Wan2.1-14B text-to-video DiT training step, Ulysses sequence parallel over all N
    GPUs of the job (one sample per SP group), parameters / optimizer state ZeRO-3 sharded over the same ranks.
    Latents 16 x 21 x 90 x 160 (75600 tokens), umT5 context 512 x 4096, synthetic N(0,1) features, bf16, activation
    checkpointing per block, AdamW.  value = samples/s of the whole job."""
    from mindspeed_mm_b200 import ops
    from mindspeed_mm_b200.api import init_distributed, stable_init_fn
    from mindspeed_mm_b200.models.diffusion import FlowMatchScheduler
    from mindspeed_mm_b200.models.wan import SoRAModel, WanConfig, WanDiT
    from mindspeed_mm_b200.ops import native
    from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig
    from mindspeed_mm_b200.parallel.state import init_parallel_state

    from mindspeed_mm_b200.parallel.state import reset_parallel_state
    ops.set_tier("native" if args.impl == "native" else "library")
    dev, rank, world = init_distributed(None)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    small = args.model == "tiny"
    steps = steps or args.steps
    cfg = WanConfig.tiny() if small else WanConfig.wan2_1_14b()
    if args.layers:
        cfg.num_layers = args.layers
    reset_parallel_state()
    ps = init_parallel_state(world_size=world, device_type=dev.type, ulysses_parallel_size=world)
    with torch.device("meta"):
        net = WanDiT(cfg)
    model = SoRAModel(net, FlowMatchScheduler(shift=5.0, sigma_min=0.0, extra_one_step=True), seed=0)
    engine = FSDPEngine(model.fsdp_units(), group=ps.get_fsdp_group() if world > 1 else False, device=dev,
                        param_dtype=torch.bfloat16, opt=OptimConfig(lr=1e-5, weight_decay=0.01), no_recompute=(),
                        comm=args.comm)
    engine.materialize(stable_init_fn(0.02, 0))
    shape = (1, cfg.in_dim, 3, 8, 8) if small else (1, cfg.in_dim, 21, 90, 160)
    g = torch.Generator().manual_seed(7)            # the same sample on every rank of the SP group
    host = [dict(latents=torch.randn(shape, generator=g).to(torch.bfloat16).pin_memory(),
                 prompt=torch.randn(1, cfg.text_len, cfg.text_dim, generator=g).to(torch.bfloat16).pin_memory())
            for _ in range(2)]
    on_dev = [{k: v.to(dev) for k, v in b.items()} for b in host]
    h2d = sum(v.numel() * v.element_size() for v in host[0].values())
    tokens = shape[2] * (shape[3] // 2) * (shape[4] // 2)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one(b):
        engine.set_lr(1e-5)
        loss = model(b, run=engine.run)
        loss.backward()
        engine.end_micro_step()
        engine.finish_step()
        return loss

    def region(batches, steps, e2e):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = native.LAUNCHES
        s.record()
        last = None
        for i in range(steps):
            b = batches[i % len(batches)]
            if e2e:
                b = {k: v.to(dev, non_blocking=True) for k, v in b.items()}
            loss = one(b)
            if e2e:
                last = float(loss.detach())
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps, native.LAUNCHES - l0, last

    region(on_dev, max(args.warmup, 3) - 1, False)
    region(host, 1, True)
    sampler = ClockSampler(local)
    sampler.start()
    torch.cuda.reset_peak_memory_stats()
    ms_dev, launches, _ = region(on_dev, steps, False)
    ms_e2e, _, loss = region(host, steps, True)
    peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
    alt = None
    if not args.no_alt and not nested:
        from mindspeed_mm_b200.api import plan_recompute_units, wan_block_activation_bytes
        torch.cuda.empty_cache()
        plan = plan_recompute_units(engine, "blocks.", wan_block_activation_bytes(cfg, -(-tokens // world)))
        region(on_dev, 1, False)
        ms_alt, _, _ = region(on_dev, steps, False)
        alt = {"recompute": f"memory-budgeted: {plan['recomputed']} of {plan['units']} blocks recomputed",
               "value": round(1e3 / ms_alt, 4), "ms_per_step": round(ms_alt, 1),
               "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}
    clocks = sampler.stop()
    if args.impl == "native":
        native.check_status()
    out = None
    if rank == 0:
        out = {"metric": "Wan2.1-14B T2V samples/s", "value": round(1e3 / ms_dev, 4), "unit": "samples/s", "n_gpus": world,
               "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_dev, 1),
               "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic (random-init weights, N(0,1) latents and text context)", "impl": args.impl,
               "config": {"model": "Wan2.1-14B T2V" if not small else "tiny", "global_batch": 1, "seq_len": tokens,
                          "parallelism": f"ulysses_sp{world} x zero3_{world}", "latent": list(shape[1:]),
                          "recompute": "activation checkpointing per block", "optimizer": "AdamW fused into backward",
                          "l2": "inputs_larger_than_L2 (28 GB of bf16 weights streamed every step)",
                          "baseline_note": "the reference publishes no Wan2.1-14B number"},
               "peak_mem_gb": round(peak_gb, 1), "clocks": clocks,
               "e2e": {"value": round(1e3 / ms_e2e, 4), "unit": "samples/s", "ms_per_step": round(ms_e2e, 1),
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": loss},
               "gpu_launches": launches, "library_fallbacks": ops.library_fallbacks()}
        if alt is not None:
            out["memory_budgeted_recompute"] = alt
    return out


def run_moe(args):
    """Third workload: Qwen3-VL-30B-A3B (128 experts, top-8) finetune step, 8192 packed tokens per GPU.  Dense parameters
    ZeRO-3 over all ranks, experts expert-parallel over all ranks (16 experts per rank on 8 GPUs) with the
    peer-memory dispatcher; AdamW in backward; activation checkpointing per layer.  value = tokens/s of the job."""
    from mindspeed_mm_b200 import ops
    from mindspeed_mm_b200.api import init_distributed, stable_init_fn
    from mindspeed_mm_b200.data.collate import batch_nbytes, to_device
    from mindspeed_mm_b200.models.qwen3_vl import Qwen3VLConfig, Qwen3VLModel
    from mindspeed_mm_b200.ops import native
    from mindspeed_mm_b200.parallel.fsdp import EngineMux, FSDPEngine, OptimConfig
    from mindspeed_mm_b200.parallel.state import init_parallel_state

    ops.set_tier("native" if args.impl == "native" else "library")
    dev, rank, world = init_distributed(None)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    small = args.model == "tiny"
    cfg = Qwen3VLConfig.tiny() if small else Qwen3VLConfig.qwen3_vl_30b_a3b()
    if args.layers:
        cfg.text.num_layers = args.layers
    cfg.text.ep_dispatcher = args.dispatcher
    ps = init_parallel_state(world_size=world, device_type=dev.type, expert_parallel_size=world)
    with torch.device("meta"):
        model = Qwen3VLModel(cfg, ep_size=world)
    opt = OptimConfig(lr=1e-5, weight_decay=0.0)
    ex = [p for _, m in model.expert_units() for p in m.parameters()]
    dense = FSDPEngine(model.fsdp_units(), group=ps.get_fsdp_group() if world > 1 else False, device=dev,
                       param_dtype=torch.bfloat16, opt=opt, exclude_params=ex, comm=args.comm)
    expert = FSDPEngine(model.expert_units(), group=False, device=dev, param_dtype=torch.bfloat16, opt=opt,
                        grad_divide=world, no_recompute=())
    mux = EngineMux(dense, expert, ep_group=ps.group("ep") if world > 1 else None)
    mux.materialize(stable_init_fn(0.02, 0))
    seq = args.seq_len if not small else 512
    host = make_batches(cfg, 2, seq, 4 if not small else 1, 2 if not small else 1, 512 if not small else 224, rank, pin=True)
    on_dev = [to_device(b, dev) for b in host]
    tokens_per_step = host[0]["n_tokens"] * world

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one(b):
        mux.set_lr(1e-5)
        loss_sum, n = model(b, run=mux.run)
        loss = loss_sum / n
        loss.backward()
        mux.end_micro_step()
        mux.finish_step()
        return loss

    def region(batches, steps, e2e):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = native.LAUNCHES
        s.record()
        last = None
        for i in range(steps):
            b = batches[i % len(batches)]
            if e2e:
                b = to_device(b, dev)
            loss = one(b)
            if e2e:
                last = float(loss.detach())
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps, native.LAUNCHES - l0, last

    region(on_dev, max(args.warmup, 3) - 1, False)
    region(host, 1, True)
    sampler = ClockSampler(local)
    sampler.start()
    ms_dev, launches, _ = region(on_dev, args.steps, False)
    ms_e2e, _, loss = region(host, args.steps, True)
    clocks = sampler.stop()
    if args.impl == "native":
        native.check_status()
    out = None
    if rank == 0:
        out = {"metric": "Qwen3-VL-30B-A3B MoE tokens/s", "value": round(tokens_per_step / (ms_dev / 1e3), 1), "unit": "tokens/s",
               "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_dev, 2),
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic (random-init weights, random text ids, U[0,1] images)", "impl": args.impl,
               "config": {"model": "Qwen3-VL-30B-A3B" if not small else "tiny", "global_batch": world, "seq_len": seq,
                          "parallelism": f"zero3_{world} (dense) x ep{world} (experts)", "dispatcher": args.dispatcher,
                          "recompute": "activation checkpointing per layer",
                          "l2": "inputs_larger_than_L2 (expert weights + optimizer state are streamed every step)"},
               "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1), "clocks": clocks,
               "e2e": {"value": round(tokens_per_step / (ms_e2e / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 2),
                       "h2d_bytes_per_step": batch_nbytes(host[0]), "d2h_bytes_per_step": 4, "last_loss": loss},
               "gpu_launches": launches, "library_fallbacks": ops.library_fallbacks()}
    return out


def _finish(out) -> int:
    """Rank 0 prints the one JSON line; every rank leaves the process group together."""
    if out is not None:
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "library", "reference"])
    ap.add_argument("--dispatcher", default="p2p", choices=["p2p", "alltoall", "allgather"], help="MoE workload only")
    ap.add_argument("--workload", default="vlm", choices=["vlm", "wan", "moe"],
                    help="vlm: Qwen2.5-VL-7B FSDP2 tokens/s (default, the driver's line); wan: Wan2.1-14B T2V samples/s")
    ap.add_argument("--model", default="qwen2_5_vl_7b", choices=["qwen2_5_vl_7b", "tiny"])
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--comm", default="auto", choices=["auto", "p2p", "nccl"])
    ap.add_argument("--recompute", default="full", choices=["full", "auto", "none"],
                    help="auto: keep the graph of as many decoder layers as free memory allows")
    ap.add_argument("--no-alt", action="store_true", help="skip the second (memory-budgeted recompute) measurement")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override decoder depth (invalidates the number)")
    ap.add_argument("--no-wan", action="store_true",
                    help="default workload only: skip the Wan2.1-14B record that the line carries on 2 or more GPUs")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "wan":
        return _finish(run_wan(args))
    if args.workload == "moe":
        return _finish(run_moe(args))

    from mindspeed_mm_b200 import ops
    from mindspeed_mm_b200.api import VLMTrainerSpec, build_vlm_trainer
    from mindspeed_mm_b200.data.collate import batch_nbytes, to_device
    from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig
    from mindspeed_mm_b200.ops import native

    ops.set_tier("native" if args.impl == "native" else "library")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    cfg = Qwen25VLConfig.qwen2_5_vl_7b() if args.model == "qwen2_5_vl_7b" else Qwen25VLConfig.tiny()
    if args.layers:
        cfg.text.num_layers = args.layers
    small = args.model == "tiny"
    spec = VLMTrainerSpec(model=cfg, lr=1e-5, weight_decay=0.0, clip_grad=0.0, train_iters=10000,
                          comm="auto" if args.comm == "auto" else args.comm, log_interval=0,
                          recompute={"full": True, "none": False, "auto": "auto"}[args.recompute],
                          tokens_per_micro_batch=args.seq_len if args.model != "tiny" else 1024)
    trainer = build_vlm_trainer(spec)
    dev = trainer.device
    seq = args.seq_len if not small else 1024
    host_batches = make_batches(cfg, 4, seq, 4 if not small else 1, 2, 448 if not small else 224, rank, pin=True)
    dev_batches = [to_device(b, dev) for b in host_batches]
    tokens_per_step = host_batches[0]["n_tokens"] * world
    h2d = batch_nbytes(host_batches[0])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def region(batches, steps, e2e):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = native.LAUNCHES
        s.record()
        last = None
        for i in range(steps):
            r = trainer.train_step([batches[i % len(batches)]])
            if e2e:
                last = float(r["loss"])        # device -> host read of the step's result
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps, native.LAUNCHES - l0, last

    # warm-up (untimed), both paths
    region(dev_batches, max(args.warmup, 3) - 1, False)
    region(host_batches, 1, True)
    sampler = ClockSampler(local)
    sampler.start()
    ms_dev, launches, _ = region(dev_batches, args.steps, False)
    ms_e2e, _, loss = region(host_batches, args.steps, True)
    peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
    # Second measurement, reported beside the headline: the same step with activation checkpointing switched off
    # for as many layers as the free memory allows (the engine's recompute="auto" plan).
    alt = None
    if args.recompute == "full" and not args.no_alt:
        from mindspeed_mm_b200.api import plan_recompute
        spec.recompute = "auto"
        torch.cuda.empty_cache()
        plan_recompute(trainer.engine, spec, world)
        region(dev_batches, 2, False)
        ms_alt, _, _ = region(dev_batches, args.steps, False)
        ms_alt_e2e, _, _ = region(host_batches, args.steps, True)
        p = trainer.engine.recompute_plan
        alt = {"recompute": f"memory-budgeted: {p['recomputed']} of {p['decoder_layers']} decoder layers and "
                            f"{p['vision_recomputed']} of {p['vision_blocks']} ViT blocks recomputed",
               "value": round(tokens_per_step / (ms_alt / 1e3), 1), "ms_per_step": round(ms_alt, 2),
               "e2e_value": round(tokens_per_step / (ms_alt_e2e / 1e3), 1),
               "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}
    clocks = sampler.stop()
    native.check_status() if args.impl == "native" else None

    plan = getattr(trainer.engine, "recompute_plan", None)
    recompute_note = ("activation checkpointing: every ViT block and decoder layer recomputed" if args.recompute == "full" else "none" if args.recompute == "none" else
                      f"memory-budgeted: {plan['recomputed']} of {plan['decoder_layers']} decoder layers recomputed, "
                      f"{plan['vision_recomputed']} of {plan['vision_blocks']} ViT blocks recomputed"
                      if plan else "full per decoder layer")
    if rank == 0:
        value = tokens_per_step / (ms_dev / 1e3)
        e2e = tokens_per_step / (ms_e2e / 1e3)
        out = {
            "metric": "Qwen2.5-VL-7B FSDP2 tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_dev, 2),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / (BASELINE_TOKENS_PER_CARD * world), 3), "dtype": "bf16",
            "data": "synthetic (random-init weights, random text ids, U[0,1] images CLIP-normalised)",
            "impl": args.impl,
            "config": {"model": "Qwen2.5-VL-7B" if not small else "tiny", "global_batch": world,
                       "seq_len": seq, "parallelism": f"fsdp{world}" if world > 1 else "single",
                       "tokens_per_gpu": host_batches[0]["n_tokens"], "images_per_gpu": 8 if not small else 2,
                       "recompute": recompute_note, "optimizer": "AdamW fp32 master+moments, fused into backward",
                       "trainable": "all parameters (ViT + merger + LLM)",
                       "l2": "inputs_larger_than_L2 (weights+optimizer state >100 GB are streamed every step)",
                       "baseline_note": "vs_baseline = value / (11042 tokens/s/card x n_gpus), the reference's "
                                        "published mcore TP=1 figure on 8x910B2; no FSDP2 number is published",
                       "comm": getattr(trainer.engine, "_p2p", None) is not None and "p2p-fused" or "nccl"},
            "peak_mem_gb": round(peak_gb, 1),
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 2),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": loss},
            "gpu_launches": launches,
            "library_fallbacks": ops.library_fallbacks(),
        }
        if alt is not None:
            out["memory_budgeted_recompute"] = alt
    else:
        out = None
    # The metric names two workloads.  Wan2.1-14B with AdamW state (14.3 B parameters x 14 bytes) does not fit one
    # 180 GB GPU, so its record rides on this line from 2 GPUs on: same process group, the VLM's memory released first.
    if world > 1 and not args.no_wan and not args.layers:
        import gc
        del trainer, dev_batches
        gc.collect()
        torch.cuda.empty_cache()
        wan = run_wan(args, steps=min(args.steps, 3), nested=True)      # 3 warm-up + 3 timed steps of 4 - 15 s each
        if out is not None:
            out["wan"] = wan
    elif out is not None:
        out["wan"] = {"unavailable": "Wan2.1-14B with optimizer state needs 200 GB: runs from 2 GPUs on"
                      if world == 1 else "skipped by flag"}
    return _finish(out)


if __name__ == "__main__":
    sys.exit(main())
