"""Generation benchmark in the VBench mould: prompt suites per dimension, several samples per prompt, one scorer per
dimension, min-max normalisation and a weighted quality / semantic total.

Reference: mindspeed_mm/tasks/evaluation/gen_impl/vbench_gen.py:27-268 (generate -> score every dimension -> table),
gen_impl/vbench_utils/compute_score.py:1-124 (dimension weights, normalisation ranges, quality : semantic = 4 : 1),
eval_datasets/datasets_vbench.py (prompt files per dimension, five samples per prompt, ``<prompt>-<k>.mp4`` naming).

Most dimensions are scored by pretrained networks (DINO, CLIP, RAFT, a detector, ...) that are not part of this package;
they plug in through ``scorers={dimension: fn(video [C, T, H, W] in [0, 1], prompt) -> float}``.  Three dimensions are
pixel statistics and ship here: temporal flickering (mean absolute frame difference), motion smoothness (how well a frame
is predicted by the mean of its neighbours) and dynamic degree (does the clip move at all).
"""
from __future__ import annotations

import csv
import json
import os
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

QUALITY = ["subject consistency", "background consistency", "temporal flickering", "motion smoothness", "aesthetic quality",
           "imaging quality", "dynamic degree"]
SEMANTIC = ["object class", "multiple objects", "human action", "color", "spatial relationship", "scene", "appearance style",
            "temporal style", "overall consistency"]
DIMENSIONS = QUALITY + SEMANTIC
WEIGHT = {d: 1.0 for d in DIMENSIONS}
WEIGHT["dynamic degree"] = 0.5
# published normalisation range of every dimension (raw score -> [0, 1])
RANGE = {"subject consistency": (0.1462, 1.0), "background consistency": (0.2615, 1.0), "temporal flickering": (0.6293, 1.0),
         "motion smoothness": (0.706, 0.9975), "dynamic degree": (0.0, 1.0), "aesthetic quality": (0.0, 1.0),
         "imaging quality": (0.0, 1.0), "object class": (0.0, 1.0), "multiple objects": (0.0, 1.0), "human action": (0.0, 1.0),
         "color": (0.0, 1.0), "spatial relationship": (0.0, 1.0), "scene": (0.0, 0.8222), "appearance style": (0.0009, 0.2855),
         "temporal style": (0.0, 0.364), "overall consistency": (0.0, 0.364)}
QUALITY_WEIGHT, SEMANTIC_WEIGHT = 4.0, 1.0
SAMPLES_PER_PROMPT = 5


# ------------------------------------------------------------------------------------------------ aggregation
def normalise(raw: Dict[str, float]) -> Dict[str, float]:
    out = {}
    for d, v in raw.items():
        lo, hi = RANGE[d]
        out[d] = (v - lo) / (hi - lo) * WEIGHT[d]
    return out


def _group(norm: Dict[str, float], dims: Sequence[str]) -> Optional[float]:
    have = [d for d in dims if d in norm]
    if not have:
        return None
    return sum(norm[d] for d in have) / sum(WEIGHT[d] for d in have)


def total_score(raw: Dict[str, float]) -> Dict[str, Optional[float]]:
    """``raw`` maps dimension -> mean raw score.  With all sixteen dimensions this is the published total; with a subset
    each group averages over the dimensions present (and the total over the groups present)."""
    unknown = [d for d in raw if d not in RANGE]
    if unknown:
        raise ValueError(f"unknown dimensions {unknown}")
    norm = normalise(raw)
    q, s = _group(norm, QUALITY), _group(norm, SEMANTIC)
    parts = [(q, QUALITY_WEIGHT), (s, SEMANTIC_WEIGHT)]
    parts = [(v, w) for v, w in parts if v is not None]
    total = sum(v * w for v, w in parts) / sum(w for _, w in parts) if parts else None
    return {"quality": q, "semantic": s, "total": total}


# ------------------------------------------------------------------------------------------------ pixel-statistic scorers
def temporal_flickering(video: torch.Tensor, _prompt=None) -> float:
    """1 - mean absolute difference of consecutive frames (on the 0..1 scale); static scenes score near 1."""
    v = video.float()
    if v.shape[1] < 2:
        return 1.0
    return float(1.0 - (v[:, 1:] - v[:, :-1]).abs().mean())


def motion_smoothness(video: torch.Tensor, _prompt=None) -> float:
    """1 - error of predicting every inner frame as the mean of its neighbours: uniform motion is smooth, jitter is not.
    (The published metric uses a learned frame interpolator as the predictor.)"""
    v = video.float()
    if v.shape[1] < 3:
        return 1.0
    mid = 0.5 * (v[:, :-2] + v[:, 2:])
    return float(1.0 - (v[:, 1:-1] - mid).abs().mean())


def dynamic_degree(video: torch.Tensor, _prompt=None, threshold: float = 0.01) -> float:
    """1.0 when the largest 5 % of per-pixel frame differences exceed ``threshold`` on average, else 0.0."""
    v = video.float().mean(0)
    if v.shape[0] < 2:
        return 0.0
    d = (v[1:] - v[:-1]).abs().flatten(1)
    k = max(1, int(0.05 * d.shape[1]))
    return float(d.topk(k, dim=1).values.mean() > threshold)


BUILTIN_SCORERS: Dict[str, Callable] = {"temporal flickering": temporal_flickering, "motion smoothness": motion_smoothness,
                                        "dynamic degree": dynamic_degree}


# ------------------------------------------------------------------------------------------------ prompts
def load_prompt_suite(path: str, dimensions: Optional[Sequence[str]] = None) -> Dict[str, List[str]]:
    """A suite is either a JSON list of ``{"prompt_en": ..., "dimension": [...]}`` records or a folder with one
    ``<dimension>.txt`` per dimension (underscores for spaces), one prompt per line."""
    suite: Dict[str, List[str]] = {}
    if os.path.isdir(path):
        for name in sorted(os.listdir(path)):
            if name.endswith(".txt"):
                dim = name[:-4].replace("_", " ")
                with open(os.path.join(path, name), encoding="utf-8") as f:
                    suite[dim] = [ln.strip() for ln in f if ln.strip()]
    else:
        with open(path, encoding="utf-8") as f:
            for rec in json.load(f):
                for dim in rec.get("dimension", []):
                    suite.setdefault(dim.replace("_", " "), []).append(rec.get("prompt_en") or rec["prompt"])
    if dimensions:
        suite = {d: suite.get(d, []) for d in dimensions}
    return suite


def sample_name(prompt: str, k: int) -> str:
    return f"{prompt}-{k}"


# ------------------------------------------------------------------------------------------------ the loop
class VideoBenchmark:
    """``generate(prompts: list[str], seed) -> list of videos [C, T, H, W] in [0, 1]``.  Ranks split the (prompt, sample)
    list; ``gather`` (e.g. ``torch.distributed.all_gather_object``) merges per-rank results."""

    def __init__(self, generate: Callable, scorers: Optional[Dict[str, Callable]] = None, samples_per_prompt: int = SAMPLES_PER_PROMPT,
                 rank: int = 0, world: int = 1, save_dir: Optional[str] = None, save_fn: Optional[Callable] = None, seed: int = 0):
        self.generate = generate
        self.scorers = dict(BUILTIN_SCORERS, **(scorers or {}))
        self.k, self.rank, self.world, self.save_dir, self.save_fn, self.seed = samples_per_prompt, rank, world, save_dir, save_fn, seed

    def run(self, suite: Dict[str, Iterable[str]], batch: int = 1, gather: Optional[Callable] = None) -> dict:
        missing = [d for d in suite if d not in self.scorers]
        if missing:
            raise ValueError(f"no scorer for dimensions {missing}; built in: {sorted(BUILTIN_SCORERS)}")
        # one generation per distinct (prompt, k); a prompt listed under several dimensions is generated once
        dims_of: Dict[str, List[str]] = {}
        for d, prompts in suite.items():
            for p in prompts:
                dims_of.setdefault(p, []).append(d)
        work = [(p, k) for p in dims_of for k in range(self.k)][self.rank::self.world]
        rows = []
        for s in range(0, len(work), batch):
            part = work[s: s + batch]
            vids = self.generate([p for p, _ in part], self.seed + s + self.rank * 100003)
            for (p, k), v in zip(part, vids):
                if self.save_dir and self.save_fn:
                    os.makedirs(self.save_dir, exist_ok=True)
                    self.save_fn(v, os.path.join(self.save_dir, sample_name(p, k)))
                for d in dims_of[p]:
                    rows.append({"dimension": d, "prompt": p, "sample": k, "score": float(self.scorers[d](v, p))})
        if gather is not None:
            rows = [r for part in gather(rows) for r in part]
        per_dim: Dict[str, List[float]] = {}
        for r in rows:
            per_dim.setdefault(r["dimension"], []).append(r["score"])
        raw = {d: sum(v) / len(v) for d, v in per_dim.items()}
        return {"dimensions": raw, "rows": rows, **total_score(raw)}

    @staticmethod
    def write_report(result: dict, out_dir: str) -> None:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "eval_result.json"), "w") as f:
            json.dump({k: v for k, v in result.items() if k != "rows"}, f, indent=2)
        with open(os.path.join(out_dir, "eval_result.csv"), "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=["dimension", "prompt", "sample", "score"])
            w.writeheader()
            w.writerows(result["rows"])
