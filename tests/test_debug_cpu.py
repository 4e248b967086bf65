"""Gradient probe, timers and the analytic parallel-plan search."""
import time

import torch

from mindspeed_mm_b200.runtime import debug as dbg


def test_grad_probe_is_identity_and_records_the_gradient(capsys):
    dbg.PROBE_LOG.clear()
    x = torch.randn(3, 4, requires_grad=True)
    w = torch.randn(4, 2)
    y = dbg.grad_probe(x * 2.0, "after_scale", keep_value=True) @ w
    y.sum().backward()
    ref = torch.ones(3, 2) @ w.t()
    assert torch.allclose(x.grad, 2.0 * ref)
    rec = dbg.PROBE_LOG[-1]
    assert rec["tag"] == "after_scale" and rec["shape"] == (3, 4) and rec["nonfinite"] == 0
    assert abs(rec["sum"] - float(ref.sum())) < 1e-4 and abs(rec["value_norm"] - float((x.detach() * 2).norm())) < 1e-4
    assert "[grad_probe] after_scale" in capsys.readouterr().out
    # another rank's probe stays silent
    dbg.PROBE_LOG.clear()
    dbg.grad_probe(x * 1.0, "other", rank=3).sum().backward()
    assert not dbg.PROBE_LOG
    z = torch.tensor([1.0, float("nan")], requires_grad=True)
    (dbg.grad_probe(z, "nan", rank=-1) * torch.tensor([1.0, float("inf")])).sum().backward()
    assert dbg.PROBE_LOG[-1]["nonfinite"] == 1


def test_timers_accumulate_and_log(capsys):
    t = dbg.Timers(cuda=False)
    for _ in range(2):
        with t("forward"):
            time.sleep(0.01)
    t("backward").start()
    time.sleep(0.005)
    t("backward").stop()
    assert t("forward").count == 2
    line = t.log(["forward", "backward", "missing"], normalizer=2.0)
    assert line.startswith("time (ms) | forward: ") and "backward: " in line and "missing: 0.00" in line
    fwd = float(line.split("forward: ")[1].split(" |")[0])
    assert 8.0 < fwd < 40.0                                          # 2 x 10 ms / 2
    assert t("forward").elapsed() == 0.0                              # log() reset the totals
    try:
        t("x").stop()
        raise AssertionError
    except RuntimeError:
        pass
    assert "time (ms)" in capsys.readouterr().out


def test_plan_search_respects_memory_and_prefers_less_communication():
    # 7 B parameters, 8192 tokens: fits on one 180 GB GPU only with sharding; plain ZeRO-3 over 8 should win
    m = dbg.ModelShape(n_params=7.6e9, n_layers=28, hidden=3584, seq_len=8192, heads=28)
    plans = dbg.suggest_parallel_plan(m, dbg.Hardware(n_gpus=8))
    assert plans and plans[0]["shard"] == 8 and plans[0]["tp"] == 1 and plans[0]["pp"] == 1 and plans[0]["ulysses"] == 1
    assert all(p["mem_gb"] <= 180.0 for p in plans)
    assert plans == sorted(plans, key=lambda r: -r["samples_per_s"])
    # one GPU cannot hold 14 B parameters with fp32 optimiser state
    assert dbg.suggest_parallel_plan(dbg.ModelShape(14e9, 40, 5120, 75600, heads=40), dbg.Hardware(n_gpus=1)) == []
    # a 75600-token sample: plans that split the sequence beat pure data parallelism, whose activations do not fit
    long_ = dbg.suggest_parallel_plan(dbg.ModelShape(14e9, 40, 5120, 75600, heads=40), dbg.Hardware(n_gpus=8), top=20)
    assert long_ and all(p["mem_gb"] <= 180.0 for p in long_)
    small_mem = dbg.suggest_parallel_plan(dbg.ModelShape(14e9, 40, 5120, 75600, heads=40), dbg.Hardware(n_gpus=8, mem_gb=60.0), top=20)
    assert small_mem and all(p["ulysses"] * p["tp"] * p["pp"] > 1 for p in small_mem)      # pure data parallel needs 65 GB
    assert small_mem[0]["ulysses"] > 1 and small_mem[0]["pp"] == 1
    # heads must divide over ulysses x tp
    assert all(28 % (p["ulysses"] * p["tp"]) == 0 for p in dbg.suggest_parallel_plan(m, dbg.Hardware(n_gpus=8), top=50))


def test_sanitize_mode_poisons_allocations_and_names_the_op():
    import torch
    from mindspeed_mm_b200 import ops
    from mindspeed_mm_b200.ops import native, sanitize
    x = torch.randn(4, 16)
    w = torch.ones(16)
    plain = ops.rms_norm
    with sanitize.debug_mode():
        assert torch.isnan(torch.empty(3, 5)).all() and torch.isnan(torch.empty_like(x)).all()
        assert int(x.new_empty(2, dtype=torch.int32)[0]) == 0x7F7F7F7F and native.SYNC_CHECK
        assert ops.rms_norm is not plain
        y = ops.rms_norm(x, w, 1e-6)                       # a healthy op passes through unchanged
        assert torch.allclose(y, plain(x, w, 1e-6))
        # an op that leaves part of its output unwritten: the hole is NaN and the wrapper names the op
        def leaky(a):
            out = torch.empty_like(a)
            out[:2] = a[:2]
            return out
        wrapped = sanitize._wrap_op("leaky", leaky)
        try:
            wrapped(x)
            raise AssertionError("the unwritten rows went unnoticed")
        except FloatingPointError as e:
            assert "ops.leaky" in str(e) and "50.00%" in str(e)
        # non-finite inputs are the caller's business
        bad_in = x.clone()
        bad_in[0, 0] = float("inf")
        ops.rms_norm(bad_in, w, 1e-6)
    assert ops.rms_norm is plain and not native.SYNC_CHECK and not torch.isnan(torch.zeros(2) + torch.empty(2).fill_(0)).any()
    assert torch.empty is not None and "alloc" not in getattr(torch.empty, "__qualname__", "")
