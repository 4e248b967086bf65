"""Optimizers, EMA, FLOPs, chunk-MBS, EP-balance planner, data-balance planner, dynamic DP/CP."""
import math

import torch

from mindspeed_mm_b200.models.qwen2_5_vl import Qwen25VLConfig
from mindspeed_mm_b200.parallel.data_balance import balance_images
from mindspeed_mm_b200.parallel.ep_balance import apply_plan, plan_duplicates
from mindspeed_mm_b200.parallel.hetero import HeteroPlan, ModulePlan, choose_dp_cp
from mindspeed_mm_b200.parallel.pp import bubble_fraction, split_layers
from mindspeed_mm_b200.runtime.features import ActivationOffload, chunk_mbs
from mindspeed_mm_b200.runtime.flops import mfu, qwen25vl_forward_flops, training_flops
from mindspeed_mm_b200.runtime.optim_extra import AdamWSwap, Muon, muon_param_groups, newton_schulz


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    g = torch.randn(32, 64)
    o = newton_schulz(g, steps=8)
    s = torch.linalg.svdvals(o)
    assert s.max() < 1.3 and s.min() > 0.5           # singular values pushed towards 1


def test_muon_and_adamw_swap_reduce_loss():
    torch.manual_seed(0)
    for make in (lambda ps: Muon(muon_param_groups(ps), lr=0.02), lambda ps: AdamWSwap([p for _, p in ps], lr=0.05)):
        lin = torch.nn.Linear(16, 16)
        x, y = torch.randn(64, 16), torch.randn(64, 16)
        opt = make(list(lin.named_parameters()))
        l0 = None
        for _ in range(30):
            loss = ((lin(x) - y) ** 2).mean()
            l0 = l0 if l0 is not None else float(loss)
            opt.zero_grad()
            loss.backward()
            opt.step()
        assert float(loss) < 0.8 * l0


def test_adamw_swap_matches_torch_adamw():
    torch.manual_seed(0)
    a, b = torch.nn.Linear(8, 8), torch.nn.Linear(8, 8)
    b.load_state_dict(a.state_dict())
    oa, ob = AdamWSwap(a.parameters(), lr=1e-2, weight_decay=0.1), torch.optim.AdamW(b.parameters(), lr=1e-2, weight_decay=0.1)
    x = torch.randn(4, 8)
    for _ in range(3):
        for m, o in ((a, oa), (b, ob)):
            o.zero_grad()
            m(x).pow(2).sum().backward()
            o.step()
    assert torch.allclose(a.weight, b.weight, atol=1e-6)


def test_chunk_mbs_equals_full():
    lin = torch.nn.Linear(8, 4)
    x = torch.randn(10, 8)
    assert torch.allclose(chunk_mbs(lin, 3)(x), lin(x), atol=1e-6)
    f = chunk_mbs(lambda a, scale=None: (a * scale, a + 1), 4, kwarg_names=("scale",))
    o1, o2 = f(x, scale=torch.arange(10.0).view(10, 1))
    assert torch.allclose(o1, x * torch.arange(10.0).view(10, 1)) and torch.allclose(o2, x + 1)


def test_activation_offload_is_identity_on_cpu():
    off = ActivationOffload()
    lin = off.wrap(torch.nn.Linear(4, 4))
    x = torch.randn(3, 4, requires_grad=True)
    lin(x).sum().backward()
    assert x.grad is not None


def test_ep_balance_plan_reduces_imbalance():
    tokens = [100, 10, 10, 10, 5, 5, 5, 5]             # expert 0 on rank 0 is hot
    plan = plan_duplicates(tokens, ep=4, max_dup=2)
    assert max(plan.loads_after) < max(plan.loads_before) and abs(sum(plan.loads_after) - sum(tokens)) < 1e-6
    assert plan.moves and plan.moves[0][0] == 0 and plan.moves[0][1] == 0
    ids = torch.zeros(100, 1, dtype=torch.long)
    out = apply_plan(ids, plan, 8)
    moved = int((out >= 8).sum())
    assert abs(moved - round(sum(m[3] for m in plan.moves if m[0] == 0) * 100)) <= 1


def test_data_balance_assignment():
    assign = balance_images([[1024, 1024, 1024, 1024], [256], [], [256, 256]])
    loads = [sum([[1024] * 4, [256], [], [256, 256]][s][i] for s, i in a) for a in assign]
    assert max(loads) <= 1536 and sum(loads) == 4 * 1024 + 3 * 256
    assert sorted(x for a in assign for x in a) == sorted([(0, 0), (0, 1), (0, 2), (0, 3), (1, 0), (3, 0), (3, 1)])


def test_dynamic_dp_cp_and_hetero_and_pp_helpers():
    assert choose_dp_cp([1000, 30000], 8, 8192) == {"cp": 4, "dp": 2}
    assert choose_dp_cp([1000, 2000], 8, 8192) == {"cp": 1, "dp": 8}
    h = HeteroPlan(8, {"vit": ModulePlan(tp=1), "llm": ModulePlan(tp=4, pp=2)})
    assert "vit: tp1 cp1 pp1 dp8" in h.describe() and "llm: tp4 cp1 pp2 dp1" in h.describe()
    assert split_layers(28, 2, [12, 16]) == [12, 16] and split_layers(10, 4) == [3, 3, 2, 2]
    assert abs(bubble_fraction(4, 8) - 3 / 11) < 1e-9 and bubble_fraction(4, 8, 2) < bubble_fraction(4, 8)


def test_flops_accounting_7b():
    cfg = Qwen25VLConfig.qwen2_5_vl_7b()
    f = qwen25vl_forward_flops(cfg, [2048] * 4, 8192)
    # ~2 * 7.6e9 params * 8192 tokens plus attention and the ViT
    assert 1.2e14 < f < 1.7e14
    assert abs(mfu(training_flops(f), 0.6, 1, 1648.3) - training_flops(f) / 0.6 / 1648.3e12) < 1e-12


def test_memory_estimate_breakdown():
    from mindspeed_mm_b200.runtime.tools import estimate_training_memory
    one = estimate_training_memory(7.6e9, shard_world=1, n_layers=28, activation_bytes_per_layer=1.5e9, workspace_gb=0, reserve_gb=0)
    assert abs(one["static_gb"] - 7.6e9 * 18 / 2 ** 30) < 1e-6 and one["gathered_units_gb"] == 0
    eight = estimate_training_memory(7.6e9, shard_world=8, n_layers=28, activation_bytes_per_layer=1.5e9, recompute_layers=28,
                                     layer_input_bytes=8192 * 3584 * 2, largest_unit_params=5.4e8, workspace_gb=0, reserve_gb=0)
    assert abs(eight["static_gb"] * 8 - one["static_gb"]) < 1e-6 and eight["gathered_units_gb"] > 0
    assert eight["activation_gb"] < one["activation_gb"] / 10 and eight["total_gb"] < 40


def test_engine_muon_matches_the_standalone_optimizer():
    """``OptimConfig(kind="muon")`` inside the sharding engine takes the same steps as ``Muon`` on plain parameters:
    orthogonalised momentum for the 2-D matrix, AdamW for the bias and the norm weight."""
    from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(16, 24)
            self.norm = torch.nn.LayerNorm(24)

        def forward(self, x):
            return self.norm(self.fc(x))

    torch.manual_seed(0)
    ref = Net()
    with torch.device("meta"):
        net = Net()
    eng = FSDPEngine([("", net)], group=False, device="cpu", param_dtype=torch.float32, no_recompute=(),
                     opt=OptimConfig(lr=0.01, weight_decay=0.1, kind="muon"))
    src = dict(ref.named_parameters())
    eng.materialize(lambda name, mod: [p.data.copy_(src[n]) for n, p in mod.named_parameters()])
    named = list(ref.named_parameters())
    groups = [dict(params=[p for n, p in named if p.dim() == 2], use_muon=True, weight_decay=0.1),
              dict(params=[p for n, p in named if p.dim() != 2], use_muon=False, weight_decay=0.0)]
    opt = Muon(groups, lr=0.01)
    x = torch.randn(8, 16)
    for _ in range(3):
        opt.zero_grad()
        ref(x).pow(2).mean().backward()
        opt.step()
        eng.set_lr(0.01)
        eng.run(net, x).pow(2).mean().backward()
        eng.end_micro_step()
        eng.finish_step()
    got = dict(eng.named_full_params())
    for n, p in ref.named_parameters():
        assert torch.allclose(got[n], p, atol=2e-5), (n, float((got[n] - p).abs().max()))   # steps are ~1e-2


def test_lr_scaling_groups_split_a_unit():
    from mindspeed_mm_b200.parallel.fsdp import FSDPEngine, OptimConfig
    with torch.device("meta"):
        net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.Linear(4, 4))
    eng = FSDPEngine([("net", net)], group=False, device="cpu", param_dtype=torch.float32, no_recompute=(),
                     opt=OptimConfig(lr=0.1, lr_scaling=((r"net\.0\.", 0.0),)))
    eng.materialize(lambda name, mod: [torch.nn.init.normal_(p, std=0.5) for p in mod.parameters()])
    before = {n: t.clone() for n, t in eng.named_full_params()}
    eng.set_lr(0.1)
    eng.run(net, torch.randn(3, 4)).pow(2).mean().backward()
    eng.end_micro_step()
    eng.finish_step()
    after = dict(eng.named_full_params())
    assert sorted(g.lr_scale for g in eng.units[0].groups) == [0.0, 1.0]
    assert torch.equal(after["net.0.weight"], before["net.0.weight"])            # multiplier 0: frozen in place
    assert not torch.equal(after["net.1.weight"], before["net.1.weight"])


def test_adaptive_clip_follows_the_norm_and_clips_outliers():
    from mindspeed_mm_b200.parallel.fsdp import AdaptiveClip, ExtremeGradientError, FSDPEngine, OptimConfig
    ac = AdaptiveClip(0.9)
    assert ac.scale_for(0.2) == 1.0 and abs(ac.avg - 0.6) < 1e-9            # first step: min(3 * norm, 1), no clipping
    for n in (0.5, 0.55, 0.45, 0.5):
        assert ac.scale_for(n) == 1.0                                       # inside mean + 3 sigma: statistics move
    avg, var = ac.avg, ac.var
    thr = avg + 3 * var ** 0.5
    s = ac.scale_for(thr * 1.5)                                             # outlier: scaled down to the threshold ...
    assert abs(s - 1 / 1.5) < 1e-9 and (ac.avg, ac.var) == (avg, var)      # ... and the statistics stay
    try:
        ac.scale_for(50.0)
        raise AssertionError("an extreme norm must stop the step")
    except ExtremeGradientError:
        pass
    # in the engine: a huge gradient after calm steps is not applied
    with torch.device("meta"):
        net = torch.nn.Linear(8, 8)
    eng = FSDPEngine([("", net)], group=False, device="cpu", param_dtype=torch.float32, no_recompute=(),
                     opt=OptimConfig(lr=0.01, clip_grad_ema_decay=0.9))
    eng.materialize(lambda name, mod: [torch.nn.init.normal_(p, std=0.3) for p in mod.parameters()])
    x = torch.randn(4, 8)
    for _ in range(3):
        eng.set_lr(0.01)
        eng.run(net, x).pow(2).mean().backward()
        eng.end_micro_step()
        eng.finish_step()
    before = {k: v.clone() for k, v in eng.named_full_params()}
    (eng.run(net, x).pow(2).mean() * 1e4).backward()
    eng.end_micro_step()
    try:
        eng.finish_step()
        raise AssertionError("expected ExtremeGradientError")
    except ExtremeGradientError:
        pass
    after = dict(eng.named_full_params())
    assert all(torch.equal(before[k], after[k]) for k in before)
