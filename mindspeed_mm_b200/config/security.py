"""Path hygiene for user-supplied file arguments: symlinks and directory traversal are reported.

Mirrors ``file_legality_checker`` / ``args_external_path_checker`` (mindspeed_mm/configs/config.py:147-256,
mindspeed_mm/utils/security_utils/validate_path.py): every path-like argument named in PATH_PARAMS is
normalised; a symlink or a path that resolves outside the allowed base is flagged (warning, not fatal).
"""
from __future__ import annotations

import os
from typing import Iterable, List, Optional, Tuple

from .tree import find_values

PATH_PARAMS = {
    "cli": ["load_base_model", "mm_data", "mm_tool", "mm_model", "profile_save_path", "tokenizer_name_or_path",
            "tensorboard_dir", "save", "load", "pretrained_checkpoint", "data_cache_path", "fsdp2_config_path"],
    "mm_model": ["from_pretrained", "ckpt_path", "model_name_or_path", "hub_backend"],
    "mm_data": ["model_name_or_path", "dataset_dir", "dataset", "cache_dir", "data_path", "data_folder",
                "from_pretrained"],
    "mm_tool": ["save_path", "profile_save_path"],
}


def normalize_path(path: str) -> Tuple[str, bool]:
    """(real path, whether any component is a symbolic link)."""
    ap = os.path.abspath(os.path.expanduser(path))
    real = os.path.realpath(ap)
    return real, real != ap and _has_link(ap)


def _has_link(path: str) -> bool:
    cur = path
    while cur and cur != os.path.dirname(cur):
        if os.path.islink(cur):
            return True
        cur = os.path.dirname(cur)
    return False


def check_path(path: str, name: str, base_dir: Optional[str] = None, warn=print) -> bool:
    """True when the path exists, is not a symlink and stays under ``base_dir`` (cwd by default)."""
    base = os.path.abspath(base_dir or os.getcwd())
    try:
        if not os.path.exists(path):
            return False
        real, is_link = normalize_path(path)
    except OSError:
        return False
    if is_link:
        warn(f"WARNING: [{name}] {path} is a symbolic link. It's normalize path is {real}")
        return False
    if not (real == base or real.startswith(base + os.sep)):
        warn(f"WARNING: [{name}] {path} attempts to traverse to an disallowed directory")
        return False
    return True


def check_args_paths(args, base_dir: Optional[str] = None, warn=print) -> List[str]:
    """Check CLI path arguments and the three config trees; returns the names that failed."""
    bad = []
    for p in PATH_PARAMS["cli"]:
        v = getattr(args, p, None)
        if v and isinstance(v, str) and os.path.exists(v) and not check_path(v, p, base_dir, warn):
            bad.append(p)
    mm = getattr(args, "mm", None)
    for tree_name, attr in (("mm_model", "model"), ("mm_data", "data"), ("mm_tool", "tool")):
        tree = getattr(mm, attr, None) if mm is not None else None
        if tree is None:
            continue
        for p in PATH_PARAMS[tree_name]:
            for v in find_values(tree, p):
                if v and isinstance(v, str) and os.path.exists(v) and not check_path(v, p, base_dir, warn):
                    bad.append(f"{tree_name}.{p}")
    return bad


def filter_input(text: str, max_len: int = 4096, allowed_extra: Iterable[str] = ()) -> str:
    """Strip control characters from free-text inputs (prompts given on the command line)."""
    keep = set(allowed_extra)
    return "".join(c for c in text[:max_len] if c.isprintable() or c in "\n\t" or c in keep)
