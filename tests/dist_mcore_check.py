"""TP x PP backend under gloo (run with torch.distributed.run, world 4 = tp 2 x pp 2, or world 2 = tp 2 / pp 2):
losses of the sharded model equal those of the single-process model with the same weights and data, for the
1F1B schedule with several micro-batches; also checks the interleaved schedule's bookkeeping with a toy stage."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from bench import make_batches  # noqa: E402
from mindspeed_mm_b200.api import stable_init_fn  # noqa: E402
from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig, Qwen25VLModel  # noqa: E402
from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig  # noqa: E402
from mindspeed_mm_b200.parallel.mcore import _stage_loss, build_mcore, shard_full_state  # noqa: E402
from mindspeed_mm_b200.parallel.pp import PipelineSchedule  # noqa: E402
from mindspeed_mm_b200.parallel.state import init_parallel_state, reset_parallel_state  # noqa: E402


def small_cfg():
    cfg = Qwen25VLConfig.tiny()
    cfg.text.num_layers = 4
    cfg.vision.depth = 2
    cfg.vision.fullatt_block_indexes = (1,)
    return cfg


def toy_interleaved(world, rank):
    """y = ((x * w0) * w1 ...) through pp*v virtual stages; loss = y.sum(); compares d loss / d w with the closed form."""
    pp, v = world, 2
    g = dist.new_group(list(range(world)))
    fg, bg = dist.new_group(list(range(world))), dist.new_group(list(range(world)))
    ws = [torch.tensor(1.0 + 0.1 * (c * pp + rank), requires_grad=True) for c in range(v)]
    mbs = [{"x": torch.full((3,), float(i + 1))} for i in range(2 * pp)]

    def stage(c, x, mb):
        x = mb["x"] if x is None else x
        y = x * ws[c]
        return y.sum() if (rank == pp - 1 and c == v - 1) else y
    sch = PipelineSchedule(stage, g, lambda mb: (3,), torch.float32, "cpu", num_chunks=v, fwd_group=fg, bwd_group=bg)
    losses = sch.run(mbs, "interleaved")
    allw = [1.0 + 0.1 * i for i in range(pp * v)]
    prod = 1.0
    for w in allw:
        prod *= w
    tot_x = sum(3.0 * (i + 1) for i in range(2 * pp))
    ok = True
    for c in range(v):
        expect = tot_x * prod / allw[c * pp + rank]
        if abs(float(ws[c].grad) - expect) > 1e-3 * abs(expect):
            ok = False
            print(f"rank {rank} toy chunk {c} grad {float(ws[c].grad)} vs {expect}")
    if rank == pp - 1 and len(losses) != 2 * pp:
        ok = False
    return ok


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    tp = 2
    pp = world // tp
    cfg = small_cfg()
    n_mb = 2 if pp > 1 else 1
    hetero = "--hetero" in sys.argv            # vision tower data parallel over the tensor-parallel ranks
    packs = make_batches(cfg, 2 * n_mb, 256, 1, 3 if hetero else 1, 112 if hetero else 224, 0, pin=False)
    ok = toy_interleaved(world, rank)
    # reference: whole model in this process
    reset_parallel_state()
    with torch.device("meta"):
        ref_model = Qwen25VLModel(cfg)
    ref = FSDPEngine(ref_model.fsdp_units(), group=False, device="cpu", param_dtype=torch.float32,
                     opt=OptimConfig(lr=1e-3), grad_accum_steps=n_mb)
    ref.materialize(stable_init_fn(0.02, 0))
    full = {n: t.detach().clone() for n, t in ref.named_full_params()}
    ref_losses = []
    for s in range(2):
        ref.set_lr(1e-3)
        ls = []
        for m in range(n_mb):
            loss_sum, n = ref_model(packs[s * n_mb + m], run=ref.run)
            (loss_sum / n).backward()
            ref.end_micro_step()
            ls.append(float((loss_sum / n).detach()))
        ref.finish_step()
        ref_losses.append(sum(ls) / n_mb)
    # sharded run
    reset_parallel_state()
    ps = init_parallel_state(world_size=world, device_type="cpu", tensor_parallel_size=tp, pipeline_parallel_size=pp)
    stage, engine, layers = build_mcore(cfg, ps, "cpu", OptimConfig(lr=1e-3), torch.float32, None, True, grad_accum_steps=n_mb,
                                        vision_data_parallel=hetero)
    engine.materialize(stable_init_fn(0.02, 0))
    local = shard_full_state(full, cfg, ps.rank_in("tp"), tp, ps.rank_in("pp"), layers)
    missing = engine.load_full_params(lambda n, shp: local.get(n))
    assert missing == [], missing
    fg = bg = None
    if pp > 1:
        groups = [None] * world
        dist.all_gather_object(groups, dist.get_process_group_ranks(ps.get_pp_group()))
        for ranks in sorted({tuple(r) for r in groups}):
            a, b = dist.new_group(list(ranks)), dist.new_group(list(ranks))
            if rank in ranks:
                fg, bg = a, b
    sch = PipelineSchedule(lambda c, x, mb: _stage_loss(stage, engine, x, mb, n_mb), ps.get_pp_group() if pp > 1 else None,
                           lambda mb: (mb["n_tokens"] // tp, cfg.text.hidden_size), torch.float32, "cpu",
                           fwd_group=fg, bwd_group=bg, after_backward=engine.end_micro_step)
    losses = []
    for s in range(2):
        engine.set_lr(1e-3)
        ls = sch.run(packs[s * n_mb:(s + 1) * n_mb])
        engine.finish_step()
        t = torch.stack(ls).mean() if ls else torch.zeros(())
        dist.all_reduce(t)
        losses.append(float(t) / tp)
    for a, b in zip(losses, ref_losses):
        if abs(a - b) > 5e-5 * max(1.0, abs(b)):
            ok = False
    flag = torch.tensor([int(ok)])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_mcore_check world={world} tp={tp} pp={pp} hetero={hetero} losses={losses} ref={ref_losses} ok={bool(flag.item())}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
