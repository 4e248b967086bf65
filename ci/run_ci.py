"""Merge gate: decides from the changed files which tiers run, then runs them.

    python ci/run_ci.py [--base origin/main] [--files changed.txt] [--gpu] [--dry-run]

* only documentation / example recipes / images changed -> nothing to run (recipes are still parsed);
* anything under the package, the tests, the entry points or the build -> build the sm_100a library and run the CPU tier
  (``pytest -m "not gpu"``; gloo for the multi-process tests);
* ``--gpu`` (a runner with B200s) -> additionally the GPU tier (``pytest -m gpu``), ``__graft_entry__.smoke()`` and the
  system-test gate (``mm-st-check compare`` of a short training log against the recorded baseline: loss 1 %, step time
  5 %, memory 10 %).

The decision rules follow the reference's gate (ci/access_control_test.py: documentation-only changes skip the test
stages; everything else runs unit tests and the system tests of the touched model families).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from typing import Iterable, List

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOC_SUFFIXES = (".md", ".rst", ".txt", ".png", ".jpg", ".gif", ".svg")
CODE_PREFIXES = ("mindspeed_mm_b200/", "tests/", "benchmarks/", "ci/", "verl_plugin/")
ROOT_CODE = ("bench.py", "__graft_entry__.py", "pyproject.toml")


def classify(path: str) -> str:
    """'doc' | 'recipe' | 'kernel' | 'code' | 'other' for one changed file."""
    if path.endswith(DOC_SUFFIXES) or path.startswith(("docs/", "profiles/")):
        return "doc"
    if path.startswith("examples/") and not path.endswith(".py"):
        return "recipe"
    if path.startswith("mindspeed_mm_b200/ops/csrc/"):
        return "kernel"
    if path.startswith(CODE_PREFIXES) or path in ROOT_CODE or (path.endswith(".py") and "/" not in path):
        return "code"
    return "other"


def plan(files: Iterable[str], gpu: bool) -> List[str]:
    kinds = {classify(f) for f in files if f.strip()}
    stages: List[str] = []
    if "recipe" in kinds:
        stages.append("recipes")
    if kinds & {"code", "kernel", "other"}:
        stages += ["build", "cpu"]
        if gpu:
            stages += ["gpu", "smoke", "st"]
    elif gpu and "kernel" in kinds:
        stages += ["build", "gpu"]
    return stages


def changed_files(base: str) -> List[str]:
    out = subprocess.run(["git", "diff", "--name-only", f"{base}...HEAD"], cwd=ROOT, capture_output=True, text=True)
    if out.returncode != 0:
        out = subprocess.run(["git", "diff", "--name-only", "HEAD~1"], cwd=ROOT, capture_output=True, text=True)
    return [l for l in out.stdout.splitlines() if l.strip()]


def _recipes_ok() -> int:
    import json
    import yaml
    bad = 0
    for d, _, names in os.walk(os.path.join(ROOT, "examples")):
        for n in names:
            p = os.path.join(d, n)
            try:
                if n.endswith((".yaml", ".yml")):
                    yaml.safe_load(open(p))
                elif n.endswith(".json"):
                    json.load(open(p))
            except Exception as e:                      # noqa: BLE001
                print(f"[ci] recipe does not parse: {p}: {e}")
                bad += 1
    return bad


COMMANDS = {
    "build": [sys.executable, "-c", "import __graft_entry__ as g; g.build()"],
    "cpu": [sys.executable, "-m", "pytest", "tests", "-x", "-q", "-m", "not gpu"],
    "gpu": [sys.executable, "-m", "pytest", "tests", "-x", "-q", "-m", "gpu"],
    "smoke": [sys.executable, "-c", "import __graft_entry__ as g; g.smoke()"],
}


def _system_tests() -> int:
    """``ci/st_cases.json``: [{"name", "recipe", "overrides": [...], "nproc", "baseline"}].  Each case trains for the few
    iterations its overrides ask for, and its log is compared with the recorded baseline (``mm-st-check record`` on the
    target machine writes one).  A case without a baseline file is reported and skipped: baselines are per machine type."""
    import json
    cases_path = os.path.join(ROOT, "ci", "st_cases.json")
    cases = json.load(open(cases_path)) if os.path.exists(cases_path) else []
    failed = 0
    for c in cases:
        base = os.path.join(ROOT, "ci", c["baseline"])
        if not os.path.exists(base):
            print(f"[ci] st case {c['name']}: no baseline at {c['baseline']} (record one with mm-st-check record), skipped")
            continue
        log = os.path.join(ROOT, "ci", f"_{c['name']}.log")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={c.get('nproc', 1)}",
               "--master-addr", "127.0.0.1", "--master-port", "29533", "-m", "mindspeed_mm_b200.runtime.trainer",
               os.path.join(ROOT, c["recipe"]), *c.get("overrides", [])]
        with open(log, "w") as f:
            rc = subprocess.run(cmd, cwd=ROOT, stdout=f, stderr=subprocess.STDOUT).returncode
        if rc == 0:
            rc = subprocess.run([sys.executable, "-m", "mindspeed_mm_b200.runtime.st_check", "compare", log, base], cwd=ROOT).returncode
        if rc != 0:
            print(f"[ci] st case {c['name']} failed")
            failed += 1
    return failed


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base", default="origin/main")
    ap.add_argument("--files", default="", help="text file with one changed path per line (default: git diff against --base)")
    ap.add_argument("--gpu", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    files = [l.strip() for l in open(a.files)] if a.files else changed_files(a.base)
    stages = plan(files, a.gpu)
    print(f"[ci] {len(files)} changed files -> stages: {stages or ['none']}")
    if a.dry_run:
        return 0
    for st in stages:
        if st == "recipes":
            if _recipes_ok():
                return 1
            continue
        if st == "st":
            if _system_tests():
                return 1
            continue
        print(f"[ci] stage {st}: {' '.join(COMMANDS[st])}", flush=True)
        rc = subprocess.run(COMMANDS[st], cwd=ROOT).returncode
        if rc != 0:
            print(f"[ci] stage {st} failed with exit code {rc}")
            return rc
    return 0


if __name__ == "__main__":
    sys.exit(main())
