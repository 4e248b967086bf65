"""Kernel-time breakdown of one training step (torch.profiler, CUDA activities only).

    python benchmarks/profile_step.py [--impl native|library] [--layers N] [--top 40] [--out FILE]

Shares only: absolute times under a profiler are not benchmark numbers.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="native")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--out", default="")
    ap.add_argument("--recompute", default="auto", choices=["full", "auto", "none"])
    ap.add_argument("--shapes", action="store_true", help="also list the costliest aten ops grouped by input shapes")
    a = ap.parse_args()
    from bench import make_batches
    from mindspeed_mm_b200 import ops
    from mindspeed_mm_b200.api import VLMTrainerSpec, build_vlm_trainer
    from mindspeed_mm_b200.data.collate import to_device
    from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig

    ops.set_tier(a.impl)
    cfg = Qwen25VLConfig.qwen2_5_vl_7b()
    if a.layers:
        cfg.text.num_layers = a.layers
    tr = build_vlm_trainer(VLMTrainerSpec(model=cfg, lr=1e-5, log_interval=0,
                                         recompute={"full": True, "none": False, "auto": "auto"}[a.recompute]))
    b = to_device(make_batches(cfg, 1, 8192, 4, 2, 448, 0, pin=True)[0], tr.device)
    for _ in range(2):
        tr.train_step([b])
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU], record_shapes=a.shapes) as prof:
        tr.train_step([b])
        torch.cuda.synchronize()
    evs = [e for e in prof.key_averages() if e.device_time_total > 0 and e.device_type.name == "CUDA"]
    if not evs:
        evs = [e for e in prof.key_averages() if e.device_time_total > 0]
    evs.sort(key=lambda e: -e.device_time_total)
    tot = sum(e.device_time_total for e in evs)
    lines = [f"total CUDA kernel time {tot / 1e3:.1f} ms (impl={a.impl}, layers={cfg.text.num_layers})"]
    for e in evs[:a.top]:
        lines.append(f"{e.device_time_total / 1e3:9.2f} ms {100 * e.device_time_total / tot:5.1f}% n={e.count:5d}  {e.key[:110]}")
    if a.shapes:
        ops_ = [e for e in prof.key_averages(group_by_input_shape=True) if e.device_time_total > 0 and e.key.startswith("aten::")]
        ops_.sort(key=lambda e: -e.device_time_total)
        lines.append("-- aten ops by input shape (device time includes children)")
        for e in ops_[:40]:
            lines.append(f"{e.device_time_total / 1e3:9.2f} ms n={e.count:5d}  {e.key:28s} {str(e.input_shapes)[:120]}")
    txt = "\n".join(lines)
    print(txt)
    if a.out:
        open(a.out, "w").write(txt + "\n")


if __name__ == "__main__":
    main()
