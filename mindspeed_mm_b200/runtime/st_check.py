"""System-test gate: turn a training log into a record and compare it with a stored baseline.

A system test runs a short training job, keeps its console log, and passes when the loss curve, the step time and the
memory footprint stay inside fixed margins of a baseline taken from an earlier good run.  The reference does this with a
log scraper and a pytest class (tests/st/test_tools/acquire_json.py:16-62, tests/st/test_tools/test_ci_st.py:8-108) that
a shell driver runs over every script of a folder (tests/st/st_run.sh); baselines are produced by
tests/st/generate_st_baseline.py.  The margins are the same here: loss 1 % relative per step, mean step time after
warm-up at most 5 % slower, allocated and peak memory at most 10 % higher.  Being faster or smaller never fails.

Command line::

    python -m mindspeed_mm_b200.runtime.st_check record  train.log  baseline.json [--warm-up 5]
    python -m mindspeed_mm_b200.runtime.st_check compare train.log  baseline.json
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional

LOSS_MARGIN = 0.01
TIME_MARGIN = 0.05
MEMORY_MARGIN = 0.10
DEFAULT_WARM_UP = 5

_NUM = r"[-+]?(?:\d+\.?\d*|\.\d+)(?:[eE][-+]?\d+)?"
_ITER = re.compile(r"iteration\s+(\d+)\s*/\s*(\d+)\s*\|(.*)")
_TIME = re.compile(r"elapsed time per iteration \(ms\):\s*(" + _NUM + ")")
_FIELD = re.compile(r"([A-Za-z][A-Za-z0-9_ ./()-]*?):\s*(" + _NUM + r"|nan|inf)\s*\|")
_MEM = re.compile(r"\[Rank (\d+)\] \(after (\d+) iterations\) memory \(MB\) \| allocated: (" + _NUM +
                  r") \| max allocated: (" + _NUM + ")")
_NOT_LOSS = ("consumed samples", "elapsed time per iteration (ms)", "learning rate", "global batch size",
             "tokens per sample", "loss scale", "grad norm", "number of skipped iterations", "number of nan iterations",
             "params norm", "throughput", "tokens per second")


@dataclass
class RunRecord:
    """What one training log says: per-step losses and step times, and each rank's memory report."""
    loss: List[float] = field(default_factory=list)
    time: List[float] = field(default_factory=list)
    memory: List[Dict[str, float]] = field(default_factory=list)
    losses: Dict[str, List[float]] = field(default_factory=dict)
    warm_up: int = DEFAULT_WARM_UP

    def to_json(self) -> dict:
        return {"warm_up": self.warm_up, "loss": self.loss, "time": self.time, "memo info": self.memory,
                "losses": self.losses}

    @classmethod
    def from_json(cls, d: dict) -> "RunRecord":
        return cls(loss=list(d.get("loss", [])), time=list(d.get("time", [])), memory=list(d.get("memo info", [])),
                   losses={k: list(v) for k, v in d.get("losses", {}).items()},
                   warm_up=int(d.get("warm_up", DEFAULT_WARM_UP)))


def parse_log(text: str, loss_key: Optional[str] = None, warm_up: int = DEFAULT_WARM_UP) -> RunRecord:
    """Scrape iteration lines and memory reports out of a console log.

    Every ``name: number |`` field of an iteration line that is not one of the bookkeeping fields counts as a loss term;
    ``loss_key`` picks the one that goes into ``loss`` (default: a field called ``loss`` or ``lm loss`` if present, else
    the first loss term)."""
    rec = RunRecord(warm_up=warm_up)
    for line in text.splitlines():
        m = _ITER.search(line)
        if m:
            tail = m.group(3)
            t = _TIME.search(tail)
            if not t:
                continue
            rec.time.append(float(t.group(1)))
            terms = {}
            for name, value in _FIELD.findall(tail):
                name = name.strip()
                if name in _NOT_LOSS:
                    continue
                terms[name] = float(value)
            for name, value in terms.items():
                rec.losses.setdefault(name, []).append(value)
            key = loss_key or next((k for k in ("loss", "lm loss") if k in terms), None) or next(iter(terms), None)
            if key is not None and key in terms:
                rec.loss.append(terms[key])
            continue
        m = _MEM.search(line)
        if m:
            rec.memory.append({"rank": int(m.group(1)), "allocated memory": float(m.group(3)),
                               "max allocated memory": float(m.group(4))})
    # keep the last report of every rank, ordered by rank
    last = {}
    for entry in rec.memory:
        last[entry["rank"]] = entry
    rec.memory = [last[r] for r in sorted(last)]
    return rec


def _exceeds(actual: float, expected: float, margin: float) -> bool:
    """True when ``actual`` is above ``expected`` by more than ``margin`` (relative)."""
    if expected == 0:
        return actual > 0
    return actual > expected and abs(actual - expected) / abs(expected) > margin


def compare(actual: RunRecord, expected: RunRecord, loss_margin: float = LOSS_MARGIN, time_margin: float = TIME_MARGIN,
            memory_margin: float = MEMORY_MARGIN, check=("loss", "time", "memory")) -> List[str]:
    """Returns the list of violations (empty = pass)."""
    problems: List[str] = []
    if "loss" in check:
        if not actual.loss:
            problems.append("no loss values in the log: the run may have failed")
        elif len(actual.loss) != len(expected.loss):
            problems.append(f"{len(actual.loss)} loss values in the log, {len(expected.loss)} in the baseline")
        else:
            for step, (a, e) in enumerate(zip(actual.loss, expected.loss), start=1):
                tol = loss_margin * abs(e)
                if not (abs(a - e) <= tol):
                    problems.append(f"loss at step {step}: {a:.6g}, baseline {e:.6g} (margin {loss_margin:.0%})")
    if "time" in check:
        w = expected.warm_up
        if len(actual.time) <= w or len(expected.time) <= w:
            problems.append(f"warm-up of {w} steps leaves no timed step ({len(actual.time)} in the log, "
                            f"{len(expected.time)} in the baseline)")
        else:
            a = sum(actual.time[w:]) / (len(actual.time) - w)
            e = sum(expected.time[w:]) / (len(expected.time) - w)
            if _exceeds(a, e, time_margin):
                problems.append(f"mean step time {a:.1f} ms, baseline {e:.1f} ms (margin {time_margin:.0%})")
    if "memory" in check and expected.memory:
        if len(actual.memory) != len(expected.memory):
            problems.append(f"memory reports of {len(actual.memory)} ranks in the log, {len(expected.memory)} in the baseline")
        else:
            for a, e in zip(actual.memory, expected.memory):
                for key in ("allocated memory", "max allocated memory"):
                    if _exceeds(a[key], e[key], memory_margin):
                        problems.append(f"rank {a['rank']} {key} {a[key]:.1f} MB, baseline {e[key]:.1f} MB "
                                        f"(margin {memory_margin:.0%})")
    return problems


def record(log_path: str, baseline_path: str, warm_up: int = DEFAULT_WARM_UP, loss_key: Optional[str] = None) -> RunRecord:
    with open(log_path, "r", encoding="utf-8", errors="replace") as f:
        rec = parse_log(f.read(), loss_key, warm_up)
    if not rec.time:
        raise ValueError(f"{log_path} has no iteration lines")
    with open(baseline_path, "w") as f:
        json.dump(rec.to_json(), f, indent=2)
    return rec


def compare_files(log_path: str, baseline_path: str, loss_key: Optional[str] = None, **margins) -> List[str]:
    with open(baseline_path) as f:
        expected = RunRecord.from_json(json.load(f))
    with open(log_path, "r", encoding="utf-8", errors="replace") as f:
        actual = parse_log(f.read(), loss_key, expected.warm_up)
    return compare(actual, expected, **margins)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("record", help="write a baseline from a log")
    r.add_argument("log")
    r.add_argument("baseline")
    r.add_argument("--warm-up", type=int, default=DEFAULT_WARM_UP)
    r.add_argument("--loss-key", default=None)
    c = sub.add_parser("compare", help="check a log against a baseline")
    c.add_argument("log")
    c.add_argument("baseline")
    c.add_argument("--loss-key", default=None)
    c.add_argument("--loss-margin", type=float, default=LOSS_MARGIN)
    c.add_argument("--time-margin", type=float, default=TIME_MARGIN)
    c.add_argument("--memory-margin", type=float, default=MEMORY_MARGIN)
    c.add_argument("--skip", nargs="*", default=[], choices=["loss", "time", "memory"])
    a = ap.parse_args(argv)
    if a.cmd == "record":
        rec = record(a.log, a.baseline, a.warm_up, a.loss_key)
        print(f"baseline with {len(rec.time)} steps written to {a.baseline}")
        return 0
    problems = compare_files(a.log, a.baseline, a.loss_key, loss_margin=a.loss_margin, time_margin=a.time_margin,
                             memory_margin=a.memory_margin,
                             check=tuple(k for k in ("loss", "time", "memory") if k not in a.skip))
    for p in problems:
        print("FAIL:", p)
    if not problems:
        print("PASS")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
