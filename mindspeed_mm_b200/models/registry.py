"""Model / dataset registries.

Counterpart of ``model_register`` / ``data_register`` (mindspeed_mm/fsdp/utils/register.py:24-61)
and ``ModelHub.build`` (mindspeed_mm/fsdp/models/modelhub.py:97): a model file registers a
builder under its ``model_id``; the trainer looks it up from the config.  ``import_plugin``
imports extra python files or packages named in ``training.plugin`` so that their decorators fire.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
from typing import Callable, Dict


class Registry:
    def __init__(self, kind: str):
        self.kind = kind
        self._items: Dict[str, Callable] = {}

    def register(self, name: str):
        def deco(obj):
            if name in self._items and self._items[name] is not obj:
                raise KeyError(f"{self.kind} {name!r} registered twice")
            self._items[name] = obj
            return obj
        return deco

    def get(self, name: str):
        if name not in self._items:
            raise KeyError(f"unknown {self.kind} {name!r}; known: {sorted(self._items)}")
        return self._items[name]

    def __contains__(self, name):
        return name in self._items

    def names(self):
        return sorted(self._items)


model_register = Registry("model")
data_register = Registry("dataset")


def import_plugin(paths) -> None:
    """Import python files / package directories / dotted modules so their registrations run."""
    for p in paths or []:
        if os.path.isdir(p):
            parent, name = os.path.split(os.path.abspath(p.rstrip("/")))
            if parent not in sys.path:
                sys.path.insert(0, parent)
            importlib.import_module(name)
        elif os.path.isfile(p):
            spec = importlib.util.spec_from_file_location(os.path.splitext(os.path.basename(p))[0], p)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        else:
            importlib.import_module(p.replace("/", "."))


def build_model(model_id: str, config, **kw):
    _ensure_builtin()
    return model_register.get(model_id)(config, **kw)


_BUILTIN_DONE = False


def _ensure_builtin():
    global _BUILTIN_DONE
    if _BUILTIN_DONE:
        return
    _BUILTIN_DONE = True
    from . import zoo  # noqa: F401  (imports every built-in model file)
