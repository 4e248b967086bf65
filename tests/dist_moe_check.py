"""Expert parallelism under gloo (run with torch.distributed.run): a tiny MoE VLM with ep = world gives the
same losses as the single-process model holding all experts, for both dispatchers; with gradient clipping the
global norm and the clip coefficient are the same on every rank and equal the single-process ones; a sharded
checkpoint of the dense + expert engines resumes to the same next loss."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from bench import make_batches  # noqa: E402
from mindspeed_mm_b200.api import stable_init_fn  # noqa: E402
from mindspeed_mm_b200.checkpoint.sharded import DistributedCheckpointer  # noqa: E402
from mindspeed_mm_b200.models.qwen3_vl import Qwen3VLConfig, Qwen3VLModel  # noqa: E402
from mindspeed_mm_b200.parallel.fsdp import EngineMux, FSDPEngine, OptimConfig  # noqa: E402
from mindspeed_mm_b200.parallel.state import init_parallel_state, reset_parallel_state  # noqa: E402


def build(cfg, world, ep, group, dispatcher, clip=0.0):
    balance = dispatcher.endswith("+balance")          # duplicate hot experts (parallel/ep_balance.py) on top of it
    dispatcher = dispatcher.split("+")[0]
    cfg.text.ep_dispatcher = dispatcher
    ps = init_parallel_state(world_size=world, device_type="cpu", expert_parallel_size=ep)
    with torch.device("meta"):
        model = Qwen3VLModel(cfg, ep_size=ep)
    opt = OptimConfig(lr=1e-3, clip_grad=clip)
    ex = [p for _, m in model.expert_units() for p in m.parameters()]
    dense = FSDPEngine(model.fsdp_units(), group=group, device="cpu", param_dtype=torch.float32, opt=opt, exclude_params=ex)
    # ep == world: experts are not sharded any further; their gradients are divided by the world size
    expert = FSDPEngine(model.expert_units(), group=False, device="cpu", param_dtype=torch.float32, opt=opt,
                        grad_divide=world, no_recompute=())
    mux = EngineMux(dense, expert, ep_group=ps.group("ep") if ep > 1 else None)
    mux.materialize(stable_init_fn(0.02, 0))
    if balance:
        for l in model.layers:
            l.mlp.experts.ep_balance_max_dup = 2
    return model, mux


def clip_and_checkpoint_check(cfg, packs, full, rank, world):
    """Clipping under EP: norm / losses equal the single-process run and are identical across ranks; then a save /
    load round trip of the muxed engines."""
    clip = 0.05                                     # far below the gradient norm: the coefficient matters
    reset_parallel_state()
    ref_model, ref = build(cfg, 1, 1, False, "alltoall", clip)
    assert ref.load_full_params(lambda n, shape: full[n]) == []
    ref.dense.grad_accum_steps = ref.expert.grad_accum_steps = world
    ref_norms, ref_losses = [], []
    for s in range(2):
        ref.set_lr(1e-3)
        ls = []
        for r in range(world):
            loss_sum, n = ref_model(packs[r][s], run=ref.run)
            (loss_sum / n).backward()
            ref.end_micro_step()
            ls.append(float((loss_sum / n).detach()))
        ref_norms.append(float(ref.finish_step()))
        ref_losses.append(sum(ls) / world)
    reset_parallel_state()
    model, mux = build(cfg, world, world, dist.group.WORLD, "alltoall", clip)
    e_local = cfg.text.num_experts // world
    getter = lambda n, shape: full[n][rank * e_local:(rank + 1) * e_local] if ".mlp.experts." in n else full[n]
    assert mux.load_full_params(getter) == []

    def step(m, eng, s):
        eng.set_lr(1e-3)
        loss_sum, n = m(packs[rank][s], run=eng.run)
        loss = loss_sum / n
        loss.backward()
        eng.end_micro_step()
        norm = eng.finish_step()
        t = loss.detach().clone()
        dist.all_reduce(t)
        return float(t) / world, norm

    ok = True
    for s in range(2):
        loss, norm = step(model, mux, s)
        norms = [torch.zeros(()) for _ in range(world)]
        dist.all_gather(norms, norm.detach().float().cpu())
        same = all(float(x) == float(norms[0]) for x in norms)
        close = abs(float(norm) - ref_norms[s]) <= 1e-4 * ref_norms[s] and abs(loss - ref_losses[s]) <= 3e-5 * max(1, abs(loss))
        ok = ok and same and close
        if rank == 0:
            print(f"dist_moe_check clip step {s}: norm {float(norm):.6f} ref {ref_norms[s]:.6f} identical_on_ranks={same} "
                  f"loss {loss:.6f} ref {ref_losses[s]:.6f}", flush=True)
    # checkpoint round trip of dense + expert shards
    root = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(root, src=0)
    ck = DistributedCheckpointer(root[0], save_async=True)
    ck.save(2, mux, {"iteration": 2})
    ck.wait()
    dist.barrier()
    reset_parallel_state()
    model2, mux2 = build(cfg, world, world, dist.group.WORLD, "alltoall", clip)
    extra = DistributedCheckpointer(root[0]).load(mux2)
    la, _ = step(model, mux, 0)
    lb, _ = step(model2, mux2, 0)
    if rank == 0:
        print(f"dist_moe_check checkpoint resume: {la:.7f} vs {lb:.7f} extra={extra}", flush=True)
    return ok and extra == {"iteration": 2} and abs(la - lb) <= 1e-6 * max(1.0, abs(la))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = Qwen3VLConfig.tiny()
    packs = [make_batches(cfg, 2, 384, 1, 1, 224, r, pin=False) for r in range(world)]
    ok = True
    # single-process twin with all experts (built first; its weights seed the EP runs)
    reset_parallel_state()
    ref_model, ref = build(cfg, 1, 1, False, "alltoall")
    full = {n: t.detach().clone() for n, t in ref.named_full_params()}
    ref.dense.grad_accum_steps = ref.expert.grad_accum_steps = world
    ref.dense.deferred = ref.expert.deferred = True
    ref_losses = []
    for s in range(2):
        ref.set_lr(1e-3)
        ls = []
        for r in range(world):
            loss_sum, n = ref_model(packs[r][s], run=ref.run)
            (loss_sum / n).backward()
            ref.end_micro_step()
            ls.append(float((loss_sum / n).detach()))
        ref.finish_step()
        ref_losses.append(sum(ls) / world)
    for disp in ("alltoall", "allgather", "alltoall+balance", "allgather+balance"):
        reset_parallel_state()
        model, mux = build(cfg, world, world, dist.group.WORLD, disp)
        e_local = cfg.text.num_experts // world

        def getter(name, shape):
            t = full[name]
            if ".mlp.experts." in name:
                t = t[rank * e_local:(rank + 1) * e_local]
            return t
        assert mux.load_full_params(getter) == []
        losses = []
        for s in range(2):
            mux.set_lr(1e-3)
            loss_sum, n = model(packs[rank][s], run=mux.run)
            loss = loss_sum / n
            loss.backward()
            mux.end_micro_step()
            mux.finish_step()
            t = loss.detach().clone()
            dist.all_reduce(t)
            losses.append(float(t) / world)
        for a, b in zip(losses, ref_losses):
            if abs(a - b) > 3e-5 * max(1, abs(b)):
                ok = False
        if disp.endswith("+balance"):           # the duplication really happened, and it evened the ranks out
            plan = model.layers[0].mlp.experts.last_balance_plan
            good = bool(plan.moves) and max(plan.loads_after) < max(plan.loads_before)
            if not good:
                print(f"rank {rank} {disp}: no rebalancing: {plan}", flush=True)
            ok = ok and good
        got = {n: t.detach().clone() for n, t in mux.named_full_params()}
        if disp == "alltoall":
            base_params = got
        else:                                   # same updated weights as the plain all-to-all run
            # splitting an expert's rows over two ranks changes the summation order of its weight gradient; Adam turns
            # the rounding of near-zero gradients into steps of a fraction of lr, so bound the largest deviation by a
            # tenth of one step and the typical one far below that
            worst = max(float((got[n] - base_params[n]).abs().max()) for n in got)
            mean = max(float((got[n] - base_params[n]).abs().mean()) for n in got)
            if worst >= 1e-4 or mean >= 1e-6:
                print(f"rank {rank} {disp}: parameters differ from the all-to-all run by {worst:.3e} (mean {mean:.3e})", flush=True)
            ok = ok and worst < 1e-4 and mean < 1e-6
        if rank == 0:
            print(f"dist_moe_check world={world} dispatcher={disp} losses={losses} ref={ref_losses}", flush=True)
    ok = clip_and_checkpoint_check(cfg, packs, full, rank, world) and ok
    flag = torch.tensor([int(ok)])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"dist_moe_check ok={bool(flag.item())}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
