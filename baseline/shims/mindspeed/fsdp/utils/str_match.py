"""Module-name patterns of the sharding / recompute / offload plans.

A pattern is a dotted module path in which one component may be ``{*}`` (any single component, e.g. a layer
index) or ``{0-3,7}`` (a list of indices and inclusive ranges).  A plain ``*`` inside a component is a
shell-style wildcard.  The match is on the whole name.
"""
import fnmatch
import re

_BRACE = re.compile(r"^\{(.*)\}$")


def _component_match(pat: str, comp: str) -> bool:
    m = _BRACE.match(pat)
    if m is None:
        return fnmatch.fnmatchcase(comp, pat) if any(c in pat for c in "*?[") else pat == comp
    body = m.group(1).strip()
    if body == "*":
        return True
    if not comp.isdigit():
        return False
    idx = int(comp)
    for part in body.split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            if int(lo) <= idx <= int(hi):
                return True
        elif int(part) == idx:
            return True
    return False


def module_name_match(pattern: str, name: str) -> bool:
    pats, comps = pattern.split("."), name.split(".")
    if len(pats) != len(comps):
        return False
    return all(_component_match(p, c) for p, c in zip(pats, comps))
