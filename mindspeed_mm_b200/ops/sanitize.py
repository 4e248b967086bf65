"""Debug mode for the native ops: poisoned outputs, per-op synchronisation and finite-output checks.

``with ops.sanitize.debug_mode():`` changes three things until the block ends:

* every buffer obtained through ``torch.empty`` / ``torch.empty_like`` / ``Tensor.new_empty`` is filled with a poison value
  (NaN for floating types, ``0x7f7f...`` for integers): a kernel that leaves part of its output unwritten no longer
  returns whatever the allocator handed back, the hole shows up as NaN;
* every native launch is followed by a device synchronise and a read of the bounded-wait status words
  (``native.SYNC_CHECK``): an asynchronous CUDA error or an expired wait is raised under the name of the op that caused it
  instead of at some later, unrelated call;
* every public function of ``mindspeed_mm_b200.ops`` checks its floating outputs: finite inputs and a non-finite output
  raise ``FloatingPointError`` naming the op and the fraction of bad elements.

This is the package's answer to what the reference gets from its sanitizer builds (device-side bounds checks and poisoned
allocations in debug libraries); the external memory checker is not available on every machine, this mode always is.
It is slow by design (a synchronise per op) and meant for bisecting a wrong loss or a hang, not for training runs.
``MM_B200_SANITIZE=1`` turns it on for a whole process (``enable()`` at import of ``mindspeed_mm_b200.ops``).
"""
from __future__ import annotations

import contextlib
import functools
import types
from typing import Callable, Dict, List, Tuple

import torch

_PATCHED: List[Tuple[object, str, object]] = []
_FLOAT = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def _poison(t: torch.Tensor) -> torch.Tensor:
    if t.numel() == 0 or t.is_meta:
        return t
    if t.dtype in _FLOAT:
        t.fill_(float("nan"))
    elif t.dtype in (torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64):
        t.fill_(0x7F if t.dtype in (torch.int8, torch.uint8) else 0x7F7F if t.dtype == torch.int16 else 0x7F7F7F7F)
    return t


def _wrap_alloc(fn: Callable) -> Callable:
    @functools.wraps(fn)
    def alloc(*a, **k):
        return _poison(fn(*a, **k))
    return alloc


def _tensors(obj):
    if isinstance(obj, torch.Tensor):
        yield obj
    elif isinstance(obj, (tuple, list)):
        for o in obj:
            yield from _tensors(o)
    elif isinstance(obj, dict):
        for o in obj.values():
            yield from _tensors(o)


def _finite(ts) -> bool:
    return all(bool(torch.isfinite(t).all()) for t in ts if t.dtype in _FLOAT and t.numel())


def _wrap_op(name: str, fn: Callable) -> Callable:
    @functools.wraps(fn)
    def op(*a, **k):
        out = fn(*a, **k)
        ins = list(_tensors(a)) + list(_tensors(k))
        for t in _tensors(out):
            if t.dtype in _FLOAT and t.numel() and not bool(torch.isfinite(t).all()):
                if _finite(ins):
                    bad = float((~torch.isfinite(t)).float().mean())
                    raise FloatingPointError(f"ops.{name}: {bad:.2%} of an output {tuple(t.shape)} {t.dtype} is not finite "
                                             f"although every input is (unwritten output region or a numerical fault)")
        return out
    op._sanitize_wrapped = fn
    return op


def enable() -> None:
    if _PATCHED:
        return
    from .. import ops
    from . import native
    for owner, attr in ((torch, "empty"), (torch, "empty_like"), (torch.Tensor, "new_empty")):
        orig = getattr(owner, attr)
        _PATCHED.append((owner, attr, orig))
        setattr(owner, attr, _wrap_alloc(orig))
    _PATCHED.append((native, "SYNC_CHECK", native.SYNC_CHECK))
    native.SYNC_CHECK = True
    skip = {"library_fallbacks", "set_tier", "get_tier", "status", "set_strict", "recompute_region", "activation_cache"}
    for name, fn in list(vars(ops).items()):
        if isinstance(fn, types.FunctionType) and not name.startswith("_") and name not in skip and fn.__module__ == ops.__name__:
            _PATCHED.append((ops, name, fn))
            setattr(ops, name, _wrap_op(name, fn))


def disable() -> None:
    while _PATCHED:
        owner, attr, orig = _PATCHED.pop()
        setattr(owner, attr, orig)


@contextlib.contextmanager
def debug_mode():
    enable()
    try:
        yield
    finally:
        disable()
