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


def config_from_dict(cfg_cls, d: dict):
    """Builds a dataclass config from a json / yaml block: unknown keys (``model_id``, ``from_pretrained`` ...) are dropped,
    lists become tuples, nested dataclass fields are built recursively, and ``preset: name`` starts from the class's
    ``name()`` factory with the remaining keys as overrides."""
    import dataclasses
    fields = {f.name: f for f in dataclasses.fields(cfg_cls)}
    known = {}
    for k, v in d.items():
        if k not in fields:
            continue
        sub = fields[k].type if isinstance(fields[k].type, type) else None
        if sub is None and isinstance(fields[k].default_factory, type):
            sub = fields[k].default_factory
        if isinstance(v, dict) and sub is not None and dataclasses.is_dataclass(sub):
            v = config_from_dict(sub, v)
        known[k] = tuple(v) if isinstance(v, list) else v
    preset = d.get("preset")
    if preset and hasattr(cfg_cls, preset):
        base = getattr(cfg_cls, preset)()
        return dataclasses.replace(base, **known)
    return cfg_cls(**known)


def build_model(model_id: str, config, **kw):
    """Instantiates a registered model.  Classes that declare ``config_class`` accept the raw config block (a dict or an
    attribute tree with ``to_dict``) in place of the dataclass."""
    _ensure_builtin()
    obj = model_register.get(model_id)
    cfg_cls = getattr(obj, "config_class", None)
    if cfg_cls is not None and config is not None and not isinstance(config, cfg_cls):
        raw = config.to_dict() if hasattr(config, "to_dict") else config
        if isinstance(raw, dict):
            config = config_from_dict(cfg_cls, raw)
    return obj(config, **kw)


_BUILTIN_DONE = False


def _ensure_builtin():
    global _BUILTIN_DONE
    if _BUILTIN_DONE:
        return
    _BUILTIN_DONE = True
    from . import zoo  # noqa: F401  (imports every built-in model file)
