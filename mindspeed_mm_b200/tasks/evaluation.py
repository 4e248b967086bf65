"""Evaluation harness: multiple-choice / VQA style benchmarks scored by exact or relaxed match.

``evaluate(generator, dataset, metric)`` runs a ``VLMGenerator``-like callable over samples of
``{"prompt_ids", "pixel_values"?, "image_grid_thw"?, "answer"}`` and aggregates accuracy across ranks; the
metric functions cover the benchmark families the reference ships (MMMU / AI2D multiple choice, DocVQA /
ChartQA relaxed accuracy: mindspeed_mm/tasks/evaluation/eval_impl/*.py, eval_datasets/*.py).
"""
from __future__ import annotations

import re
from typing import Callable, Dict, Iterable, List

import torch
import torch.distributed as dist


def multiple_choice_match(pred: str, answer: str) -> bool:
    m = re.search(r"\b([A-H])\b", pred.strip().upper())
    return bool(m) and m.group(1) == answer.strip().upper()


def exact_match(pred: str, answer: str) -> bool:
    norm = lambda s: re.sub(r"[^a-z0-9 ]", "", s.lower()).strip()      # noqa: E731
    return norm(pred) == norm(answer)


def relaxed_accuracy(pred: str, answer: str, tol: float = 0.05) -> bool:
    """ChartQA-style: numeric answers within 5 %, otherwise exact match."""
    try:
        p, a = float(pred.strip().rstrip("%")), float(answer.strip().rstrip("%"))
        return abs(p - a) <= tol * abs(a) if a != 0 else p == a
    except ValueError:
        return exact_match(pred, answer)


def anls(pred: str, answers: List[str], threshold: float = 0.5) -> float:
    """Average normalised Levenshtein similarity (DocVQA)."""
    def lev(a, b):
        dp = list(range(len(b) + 1))
        for i, ca in enumerate(a, 1):
            prev, dp[0] = dp[0], i
            for j, cb in enumerate(b, 1):
                prev, dp[j] = dp[j], min(dp[j] + 1, dp[j - 1] + 1, prev + (ca != cb))
        return dp[-1]
    best = 0.0
    for a in answers:
        p_, a_ = pred.strip().lower(), a.strip().lower()
        d = lev(p_, a_) / max(len(p_), len(a_), 1)
        best = max(best, 1 - d if d < threshold else 0.0)
    return best


def _anls_any(pred: str, answer) -> float:
    return anls(pred, list(answer) if isinstance(answer, (list, tuple)) else [answer])


METRICS: Dict[str, Callable] = {"multiple_choice": multiple_choice_match, "exact_match": exact_match,
                                "relaxed_accuracy": relaxed_accuracy, "anls": _anls_any}


def evaluate(predict: Callable[[dict], str], samples: Iterable[dict], metric: str = "exact_match") -> Dict[str, float]:
    fn = METRICS[metric]
    hit, n = 0.0, 0
    cats: Dict[str, List[float]] = {}
    for s in samples:
        score = float(fn(predict(s), s["answer"]))
        hit += score
        n += 1
        if "category" in s:
            c = cats.setdefault(s["category"], [0.0, 0])
            c[0] += score
            c[1] += 1
    if cats and not (dist.is_initialized() and dist.get_world_size() > 1):
        per = {k: v[0] / v[1] for k, v in sorted(cats.items())}
        return {"accuracy": hit / max(n, 1), "n": n, "per_category": per}
    t = torch.tensor([hit, n], dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size() > 1:
        if torch.cuda.is_available() and dist.get_backend() == "nccl":
            t = t.cuda()
        dist.all_reduce(t)
    return {"accuracy": float(t[0] / max(t[1], 1)), "n": int(t[1])}
