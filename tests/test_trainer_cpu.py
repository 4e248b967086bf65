"""YAML-driven trainer end to end on CPU, sampler resume, packing, watchdog."""
import os
import re
import time

import torch

from mindspeed_mm_b200.config import load_config
from mindspeed_mm_b200.data.packing import DynamicBatcher, balance_across_ranks, greedy_pack
from mindspeed_mm_b200.data.samplers import BaseRandomBatchSampler
from mindspeed_mm_b200.runtime.logging import format_training_log
from mindspeed_mm_b200.runtime.lr_scheduler import LRSchedule
from mindspeed_mm_b200.runtime.tools import Watchdog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_trainer_yaml_cpu(tmp_path, capsys):
    from mindspeed_mm_b200.runtime.trainer import Trainer
    args = load_config(os.path.join(ROOT, "examples/qwen2.5vl/tiny_native.yaml"),
                       ["training.train_iters=3", "model.config.text.num_layers=1", "model.config.vision.depth=1",
                        "model.config.vision.fullatt_block_indexes=[0]", f"training.save={tmp_path}/ck",
                        "training.save_interval=2", "data.dataset_param.basic_parameters.seq_len=300",
                        "data.dataset_param.basic_parameters.images_per_sample=1", "training.micro_batch_size=1"],
                       world_size=1)
    tr = Trainer(args, device="cpu")
    hist = tr.train()
    assert len(hist) == 3 and all(h["loss"] == h["loss"] for h in hist)
    out = capsys.readouterr().out
    # the scraped fields of the reference's log line
    m = re.search(r"iteration\s+3/\s+3 \| consumed samples:\s+3 \| elapsed time per iteration \(ms\): ([\d.]+) \|"
                  r" learning rate: ([\d.E+-]+) \| global batch size:\s+1 \| tokens per sample: ([\d.]+) \| loss: ", out)
    assert m, out
    assert os.path.exists(tmp_path / "ck" / "iter_0000002") and \
        open(tmp_path / "ck" / "latest_checkpointed_iteration.txt").read() == "2"
    # resume: iteration and sampler state come back
    args2 = load_config(os.path.join(ROOT, "examples/qwen2.5vl/tiny_native.yaml"),
                        ["training.train_iters=3", "model.config.text.num_layers=1", "model.config.vision.depth=1",
                         "model.config.vision.fullatt_block_indexes=[0]", f"training.save={tmp_path}/ck",
                         f"training.load={tmp_path}/ck", "training.load_format=dcp",
                         "data.dataset_param.basic_parameters.seq_len=300",
                         "data.dataset_param.basic_parameters.images_per_sample=1", "training.micro_batch_size=1"],
                        world_size=1)
    tr2 = Trainer(args2, device="cpu")
    assert tr2.train_engine.iteration == 2 and tr2.train_engine.consumed_train_samples == 2
    h2 = tr2.train()
    assert len(h2) == 1 and abs(h2[0]["loss"] - hist[2]["loss"]) < 1e-4


def test_sampler_resume_is_exact():
    a = BaseRandomBatchSampler(37, 2, dp_rank=1, dp_world=2, seed=3)
    it = iter(a)
    first = [next(it) for _ in range(5)]
    state = a.state_dict()
    nxt = [next(it) for _ in range(6)]
    b = BaseRandomBatchSampler(37, 2, dp_rank=1, dp_world=2, seed=3)
    b.load_state_dict(state)
    assert [next(iter(b)) for _ in range(1)][0] == nxt[0]
    # ranks see disjoint samples in one epoch
    r0 = BaseRandomBatchSampler(16, 2, 0, 2, seed=1)
    r1 = BaseRandomBatchSampler(16, 2, 1, 2, seed=1)
    i0, i1 = iter(r0), iter(r1)
    s0 = sum((next(i0) for _ in range(4)), [])
    s1 = sum((next(i1) for _ in range(4)), [])
    assert not set(s0) & set(s1) and len(set(s0 + s1)) == 16


def test_packing_and_balance():
    bins = greedy_pack([900, 300, 700, 100, 50, 1000], 1024)
    assert sorted(sum(bins, [])) == list(range(6))
    assert all(sum([900, 300, 700, 100, 50, 1000][i] for i in b) <= 1024 for b in bins)
    samples = [{"input_ids": [0] * n} for n in (500, 600, 400, 100, 300)]
    out = list(DynamicBatcher(samples, 1000, buffer_size=3))
    assert sum(len(b) for b in out) == 5 and all(sum(len(s["input_ids"]) for s in b) <= 1000 for b in out)
    parts = balance_across_ranks([8, 7, 6, 5, 4], 2)
    loads = [sum([8, 7, 6, 5, 4][i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 4 and sorted(sum(parts, [])) == [0, 1, 2, 3, 4]


def test_lr_schedule_shapes():
    s = LRSchedule(lr=1e-3, train_iters=100, lr_decay_style="cosine", lr_warmup_ratio=0.1, lr_min=1e-5)
    assert s(0) == 0.0 and abs(s(5) - 5e-4) < 1e-12 and abs(s(10) - 1e-3) < 1e-12
    assert abs(s(100) - 1e-5) < 1e-9 and s(55) < s(20)
    lin = LRSchedule(lr=1e-3, train_iters=100, lr_decay_style="linear", lr_warmup_steps=0, lr_min=1e-4)
    assert abs(lin(50) - 5e-4) < 1e-12 and abs(lin(99) - 1e-4) < 1e-12
    assert LRSchedule(lr=1e-3, train_iters=10, lr_decay_style="constant")(7) == 1e-3


def test_log_line_format():
    s = format_training_log(7, 100, 56, 0.1234, 1e-5, 8, {"loss": 2.5}, grad_norm=1.25, tokens_per_sample=8192.0)
    assert "iteration        7/     100 |" in s and "elapsed time per iteration (ms): 123.4 |" in s
    assert "learning rate: 1.000000E-05 |" in s and "global batch size:     8 |" in s
    assert "tokens per sample: 8192.0 |" in s and "loss: 2.500000E+00 |" in s and "grad norm: 1.250 |" in s


def test_watchdog_fires_on_stall_and_not_on_progress():
    hits = []
    w = Watchdog(0.3, on_timeout=lambda it, idle: hits.append(it), poll_s=0.05).start()
    for i in range(5):
        w.beat(i)
        time.sleep(0.1)
    assert not hits
    time.sleep(0.6)       # a rank that stops beating (hung step) is detected on the host
    assert hits == [4] and w.fired
    w.stop()


def test_trainer_runs_speech_lm_recipes(capsys):
    import pytest
    from mindspeed_mm_b200.runtime.trainer import Trainer
    for rel in ("examples/moss_tts/finetune_moss_tts_delay_tiny.yaml", "examples/cosyvoice3/finetune_cosyvoice3_tiny.yaml",
                "examples/qwen3tts/finetune_qwen3tts_tiny.yaml", "examples/ltx2/finetune_ltx2_tiny.yaml"):
        args = load_config(os.path.join(ROOT, rel), ["training.train_iters=3"], world_size=1)
        hist = Trainer(args, device="cpu").train()
        assert len(hist) == 3 and all(h["loss"] == h["loss"] and h["loss"] > 0 for h in hist), rel


def test_training_loop_stops_when_a_kernel_reported_a_timeout():
    """The loop reads the kernels' status word at every iteration boundary; a non-zero word (a bounded device wait
    expired during the step) ends the run before the next step instead of training on incomplete tensors."""
    import pytest
    from mindspeed_mm_b200.runtime.train_engine import NativeKernelTimeout
    from mindspeed_mm_b200.runtime.trainer import Trainer
    args = load_config(os.path.join(ROOT, "examples/qwen2.5vl/tiny_native.yaml"),
                       ["training.train_iters=4", "model.config.text.num_layers=1", "model.config.vision.depth=1",
                        "model.config.vision.fullatt_block_indexes=[0]",
                        "data.dataset_param.basic_parameters.seq_len=300",
                        "data.dataset_param.basic_parameters.images_per_sample=1", "training.micro_batch_size=1"],
                       world_size=1)
    tr = Trainer(args, device="cpu")
    word = torch.zeros(1, dtype=torch.int32)
    tr.train_engine.status_word = word
    real_step = tr.train_engine.train_step

    def step_with_timeout(mbs):
        r = real_step(mbs)
        if tr.train_engine.iteration == 2:       # what a kernel does when its wait runs out
            word.fill_(2)
        return r
    tr.train_engine.train_step = step_with_timeout
    with pytest.raises(NativeKernelTimeout) as ei:
        tr.train()
    assert ei.value.exit_code == 3 and "status 2" in str(ei.value)
    assert tr.train_engine.iteration == 2 and len(tr.train_engine.history) == 1   # the bad step is not logged as done
    assert int(word) == 0                                                        # cleared for a restart in-process


def test_trainer_keeps_and_restores_a_moving_average(tmp_path):
    """``training.use_ema``: the average follows the master weights with the configured decay, is written with the
    checkpoint's per-rank state and comes back on resume; ``swap`` exchanges it with the live weights."""
    from mindspeed_mm_b200.runtime.trainer import Trainer
    base = ["model.config.text.num_layers=1", "model.config.vision.depth=1", "model.config.vision.fullatt_block_indexes=[0]",
            "data.dataset_param.basic_parameters.seq_len=300", "data.dataset_param.basic_parameters.images_per_sample=1",
            "training.micro_batch_size=1", "training.use_ema=true", "training.ema_decay=0.5", "training.lr=1.0e-3",
            f"training.save={tmp_path}/ck"]
    cfg = os.path.join(ROOT, "examples/qwen2.5vl/tiny_native.yaml")
    tr = Trainer(load_config(cfg, base + ["training.train_iters=1", "training.save_interval=1"], world_size=1), device="cpu")
    ema = tr.train_engine.ema
    g0 = tr.engine.units[-1].groups[0]
    w0 = g0.master.clone()
    tr.train()
    w1 = g0.master.clone()
    assert ema.steps == 1 and not torch.equal(w1, w0)
    s = ema.shadow[-1].clone()
    assert torch.allclose(s, 0.5 * w0 + 0.5 * w1, atol=1e-7)
    ema.swap()                                                              # master now holds the average
    assert torch.allclose(g0.master, s) and torch.allclose(ema.shadow[-1], w1)
    ema.swap()
    assert torch.allclose(g0.master, w1)
    tr2 = Trainer(load_config(cfg, base + ["training.train_iters=1", f"training.load={tmp_path}/ck"], world_size=1), device="cpu")
    assert tr2.train_engine.ema.steps == 1
    assert torch.allclose(tr2.train_engine.ema.shadow[-1], s)


def test_scalars_go_to_tensorboard_and_offline_wandb(tmp_path):
    """``tools.tensorboard_dir`` / ``tools.wandb_project``: loss, learning rate, gradient norm and the MoE router's auxiliary
    loss per iteration, each also against the consumed samples."""
    import json
    from tensorboard.backend.event_processing.event_accumulator import EventAccumulator
    from mindspeed_mm_b200.runtime.trainer import Trainer
    args = load_config(os.path.join(ROOT, "examples/qwen3vl/tiny_moe_native.yaml"),
                       ["parallel.expert_parallel_size=1", "training.train_iters=2", "training.clip_grad=1.0",
                        "model.config.text.router_aux_loss_coef=0.01", "data.dataset_param.basic_parameters.seq_len=200",
                        "data.dataloader_param.pin_memory=false", f"tools.tensorboard_dir={tmp_path}/tb",
                        "tools.wandb_project=demo", f"tools.wandb_save_dir={tmp_path}/wb"], world_size=1)
    hist = Trainer(args, device="cpu").train()
    assert "load_balancing_loss" in hist[-1] and hist[-1]["load_balancing_loss"] > 0
    acc = EventAccumulator(str(tmp_path / "tb"))
    acc.Reload()
    tags = set(acc.Tags()["scalars"])
    assert {"lm loss", "lm loss vs samples", "learning-rate", "grad-norm", "load_balancing_loss"} <= tags
    assert [e.step for e in acc.Scalars("lm loss")] == [1, 2]
    rows = [json.loads(l) for l in open(tmp_path / "wb" / "wandb-offline.jsonl")]
    assert [r["iteration"] for r in rows] == [1, 2] and abs(rows[1]["lm loss"] - hist[1]["loss"]) < 1e-6
