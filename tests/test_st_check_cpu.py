"""The system-test gate: log scraping and baseline comparison (thresholds of tests/st/test_tools/test_ci_st.py:11-13)."""
import json

from mindspeed_mm_b200.runtime import st_check
from mindspeed_mm_b200.runtime.logging import format_training_log


def _log(losses, times, mem=(100.0, 200.0)):
    lines = ["some banner"]
    for i, (l, t) in enumerate(zip(losses, times), start=1):
        lines.append(format_training_log(i, len(losses), i * 8, t / 1000.0, 1e-5, 8, {"loss": l, "aux": 0.5 * l},
                                         grad_norm=1.25, tokens_per_sample=1024.0))
    lines.append(f"[Rank 0] (after {len(losses)} iterations) memory (MB) | allocated: {mem[0]} | max allocated: {mem[1]} | "
                 f"reserved: 1 | max reserved: 2")
    return "\n".join(lines)


def test_parse_log_reads_formatter_output():
    rec = st_check.parse_log(_log([2.0, 1.5, 1.25], [900.0, 500.0, 510.0]), warm_up=1)
    assert rec.loss == [2.0, 1.5, 1.25]
    assert rec.time == [900.0, 500.0, 510.0]
    assert rec.losses["aux"] == [1.0, 0.75, 0.625]
    assert "grad norm" not in rec.losses and "learning rate" not in rec.losses
    assert rec.memory == [{"rank": 0, "allocated memory": 100.0, "max allocated memory": 200.0}]


def test_compare_margins():
    base = st_check.parse_log(_log([2.0, 1.5, 1.25], [900.0, 500.0, 500.0]), warm_up=1)
    same = st_check.parse_log(_log([2.0, 1.5, 1.25 * 1.005], [2000.0, 510.0, 520.0], mem=(105.0, 215.0)), warm_up=1)
    assert st_check.compare(same, base) == []
    faster = st_check.parse_log(_log([2.0, 1.5, 1.25], [900.0, 100.0, 100.0], mem=(10.0, 20.0)), warm_up=1)
    assert st_check.compare(faster, base) == []
    bad = st_check.parse_log(_log([2.0, 1.6, 1.25], [900.0, 560.0, 560.0], mem=(100.0, 230.0)), warm_up=1)
    problems = st_check.compare(bad, base)
    assert len(problems) == 3
    assert any("loss at step 2" in p for p in problems)
    assert any("mean step time" in p for p in problems)
    assert any("max allocated memory" in p for p in problems)
    short = st_check.parse_log(_log([2.0], [900.0]), warm_up=1)
    assert any("loss values" in p for p in st_check.compare(short, base))


def test_record_and_compare_cli(tmp_path):
    log = tmp_path / "train.log"
    log.write_text(_log([3.0, 2.0, 1.0, 0.5], [800.0, 400.0, 400.0, 400.0]))
    base = tmp_path / "base.json"
    assert st_check.main(["record", str(log), str(base), "--warm-up", "1"]) == 0
    stored = json.loads(base.read_text())
    assert stored["warm_up"] == 1 and stored["loss"] == [3.0, 2.0, 1.0, 0.5]
    assert st_check.main(["compare", str(log), str(base)]) == 0
    slow = tmp_path / "slow.log"
    slow.write_text(_log([3.0, 2.0, 1.0, 0.5], [800.0, 500.0, 500.0, 500.0]))
    assert st_check.main(["compare", str(slow), str(base)]) == 1
    assert st_check.main(["compare", str(slow), str(base), "--skip", "time"]) == 0


def test_trainer_log_passes_its_own_baseline(tmp_path, capsys):
    """A short run is recorded as a baseline; a second run with the same seed must reproduce its loss curve."""
    import os
    from mindspeed_mm_b200.config import load_config
    from mindspeed_mm_b200.runtime.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    over = ["training.train_iters=3", "model.config.text.num_layers=1", "model.config.vision.depth=1",
            "model.config.vision.fullatt_block_indexes=[0]", "data.dataset_param.basic_parameters.seq_len=300",
            "data.dataset_param.basic_parameters.images_per_sample=1", "training.micro_batch_size=1"]
    logs = []
    for _ in range(2):
        args = load_config(os.path.join(root, "examples/qwen2.5vl/tiny_native.yaml"), over, world_size=1)
        hist = Trainer(args, device="cpu").train()
        logs.append((capsys.readouterr().out, hist))
    (tmp_path / "a.log").write_text(logs[0][0])
    (tmp_path / "b.log").write_text(logs[1][0])
    rec = st_check.record(str(tmp_path / "a.log"), str(tmp_path / "base.json"), warm_up=1)
    assert len(rec.loss) == 3 and all(abs(a - h["loss"]) <= 1e-5 * abs(h["loss"]) for a, h in zip(rec.loss, logs[0][1]))
    assert st_check.compare_files(str(tmp_path / "b.log"), str(tmp_path / "base.json"), check=("loss", "memory")) == []


def test_merge_gate_stage_selection():
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("run_ci", os.path.join(root, "ci", "run_ci.py"))
    ci = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ci)
    assert ci.classify("docs/migration.md") == "doc" and ci.classify("examples/qwen3vl/tiny_moe_native.yaml") == "recipe"
    assert ci.classify("mindspeed_mm_b200/ops/csrc/gemm.cu") == "kernel" and ci.classify("bench.py") == "code"
    assert ci.plan(["README.md", "profiles/x.md"], gpu=True) == []
    assert ci.plan(["examples/a/b.yaml", "docs/x.md"], gpu=False) == ["recipes"]
    assert ci.plan(["mindspeed_mm_b200/parallel/fsdp.py"], gpu=False) == ["build", "cpu"]
    assert ci.plan(["mindspeed_mm_b200/ops/csrc/gemm.cu", "README.md"], gpu=True) == ["build", "cpu", "gpu", "smoke", "st"]
    assert ci._recipes_ok() == 0                       # every committed recipe parses
    assert ci.main(["--files", os.devnull, "--dry-run"]) == 0
