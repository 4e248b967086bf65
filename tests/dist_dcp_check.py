"""torch-DCP training checkpoints under gloo (run with torch.distributed.run): two ranks train a step, save (sync or
--async), train one more step and print its loss; the caller resumes the checkpoint with another world size."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from bench import make_batches  # noqa: E402
from mindspeed_mm_b200.api import stable_init_fn  # noqa: E402
from mindspeed_mm_b200.checkpoint import hf as hfio  # noqa: E402
from mindspeed_mm_b200.checkpoint.dcp import TorchDCPCheckpointer  # noqa: E402
from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel  # noqa: E402
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig  # noqa: E402


def small_cfg():
    cfg = Qwen25VLConfig.tiny()
    cfg.text.num_layers, cfg.vision.depth, cfg.vision.fullatt_block_indexes = 1, 1, (0,)
    return cfg


def build(cfg, group):
    with torch.device("meta"):
        m = Qwen25VLModel(cfg)
    e = FSDPEngine(m.fsdp_units(), group=group, device="cpu", param_dtype=torch.float32, opt=OptimConfig(lr=1e-3))
    e.materialize(stable_init_fn(0.02, 0))
    return m, e


def step(m, e, b):
    e.set_lr(1e-3)
    ls, n = m(b, run=e.run)
    loss = ls / n
    loss.backward()
    e.end_micro_step()
    e.finish_step()
    return float(loss.detach())


def main():
    out_dir = sys.argv[1]
    dist.init_process_group("gloo")
    cfg = small_cfg()
    b = make_batches(cfg, 2, 300, 1, 1, 224, 0, pin=False)           # the same packs on every rank
    m, e = build(cfg, dist.group.WORLD)
    step(m, e, b[0])
    ck = TorchDCPCheckpointer(out_dir, ops=hfio.qwen25vl_ops(cfg), save_async="--async" in sys.argv)
    ck.save(1, e, {"iteration": 1, "consumed_train_samples": 2})
    ck.wait()
    nxt = step(m, e, b[1])
    if dist.get_rank() == 0:
        print(f"dist_dcp_check world={dist.get_world_size()} next_loss={nxt:.8f} ok=True", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
