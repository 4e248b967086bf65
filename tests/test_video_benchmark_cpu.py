"""Generation benchmark: aggregation arithmetic, pixel-statistic scorers, the generate -> score -> report loop."""
import json

import torch

from mindspeed_mm_b200.tasks import video_benchmark as vb


def test_total_score_arithmetic():
    raw = {d: vb.RANGE[d][1] for d in vb.DIMENSIONS}                 # every dimension at the top of its range
    r = vb.total_score(raw)
    assert abs(r["quality"] - 1.0) < 1e-9 and abs(r["semantic"] - 1.0) < 1e-9 and abs(r["total"] - 1.0) < 1e-9
    raw = {d: vb.RANGE[d][0] for d in vb.DIMENSIONS}
    assert abs(vb.total_score(raw)["total"]) < 1e-9
    mid = {d: 0.5 * (vb.RANGE[d][0] + vb.RANGE[d][1]) for d in vb.DIMENSIONS}
    mid.update({d: vb.RANGE[d][1] for d in vb.SEMANTIC})
    r = vb.total_score(mid)
    assert abs(r["quality"] - 0.5) < 1e-9 and abs(r["total"] - (4 * 0.5 + 1.0) / 5) < 1e-9
    # dynamic degree counts half inside the quality group
    only = vb.total_score({"dynamic degree": 1.0, "imaging quality": 0.0})
    assert abs(only["quality"] - 0.5 / 1.5) < 1e-9 and only["semantic"] is None and only["total"] == only["quality"]
    try:
        vb.total_score({"made up": 1.0})
        raise AssertionError("unknown dimension accepted")
    except ValueError:
        pass


def _moving(T=8, step=2, jitter=0.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    base = torch.rand(3, 32, 64, generator=g)
    frames = [torch.roll(base, shifts=step * t + (int(jitter * (t % 2))), dims=2) for t in range(T)]
    return torch.stack(frames, 1)


def test_pixel_statistic_scorers_order_clips_sensibly():
    still = torch.rand(3, 1, 16, 16).expand(3, 6, 16, 16)
    assert vb.temporal_flickering(still) == 1.0 and vb.motion_smoothness(still) == 1.0 and vb.dynamic_degree(still) == 0.0
    smooth = torch.linspace(0, 1, 8).view(1, 8, 1, 1).expand(3, 8, 4, 4)              # linear fade: perfectly predictable
    assert abs(vb.motion_smoothness(smooth) - 1.0) < 1e-6 and vb.temporal_flickering(smooth) < 1.0
    noise = torch.rand(3, 8, 16, 16)
    assert vb.motion_smoothness(noise) < 0.8 and vb.temporal_flickering(noise) < 0.8 and vb.dynamic_degree(noise) == 1.0
    assert vb.dynamic_degree(_moving()) == 1.0
    assert vb.temporal_flickering(torch.rand(3, 1, 4, 4)) == 1.0                       # single frame


def test_benchmark_loop_splits_ranks_and_writes_report(tmp_path):
    (tmp_path / "suite").mkdir()
    (tmp_path / "suite" / "temporal_flickering.txt").write_text("a still lake\na busy street\n")
    (tmp_path / "suite" / "dynamic_degree.txt").write_text("a busy street\n")
    suite = vb.load_prompt_suite(str(tmp_path / "suite"))
    assert suite == {"dynamic degree": ["a busy street"], "temporal flickering": ["a still lake", "a busy street"]}
    calls = []

    def generate(prompts, seed):
        calls.append(list(prompts))
        return [torch.rand(3, 1, 8, 8).expand(3, 4, 8, 8) if "still" in p else torch.rand(3, 4, 8, 8) for p in prompts]

    saved = []
    parts = []
    for rank in range(2):
        bench = vb.VideoBenchmark(generate, samples_per_prompt=3, rank=rank, world=2, save_dir=str(tmp_path / "vid"),
                                  save_fn=lambda v, path: saved.append(path))
        parts.append(bench.run(suite, batch=2)["rows"])
    assert sum(len(c) for c in calls) == 2 * 3                       # the shared prompt is generated once per sample index
    assert len(saved) == 6 and sorted(saved)[3].endswith("a still lake-0") and sorted(saved)[0].endswith("a busy street-0")
    merged = vb.VideoBenchmark(generate, samples_per_prompt=3).run(suite, gather=lambda rows: parts)
    assert len(merged["rows"]) == 3 * 3                              # 2 prompts x flickering + 1 prompt x dynamic degree, 3 samples
    assert merged["dimensions"]["dynamic degree"] == 1.0 and 0.5 < merged["dimensions"]["temporal flickering"] < 1.0
    assert merged["semantic"] is None and merged["total"] == merged["quality"]
    vb.VideoBenchmark.write_report(merged, str(tmp_path / "out"))
    rep = json.loads((tmp_path / "out" / "eval_result.json").read_text())
    assert set(rep) == {"dimensions", "quality", "semantic", "total"}
    assert (tmp_path / "out" / "eval_result.csv").read_text().count("\n") == 10
    js = tmp_path / "full.json"
    js.write_text(json.dumps([{"prompt_en": "a cat", "dimension": ["object_class", "color"]}]))
    assert vb.load_prompt_suite(str(js)) == {"object class": ["a cat"], "color": ["a cat"]}
    try:
        vb.VideoBenchmark(generate).run({"color": ["a cat"]})
        raise AssertionError("a dimension without a scorer must be refused")
    except ValueError:
        pass
