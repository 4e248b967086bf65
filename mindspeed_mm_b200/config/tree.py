"""Attribute tree over nested dicts (``args.mm.model.image_encoder.vision_encoder.hidden_size``).

Same access pattern as the reference's ``ConfigReader`` (mindspeed_mm/configs/config.py:10-64): dict
values become nodes, ``dtype`` strings become torch dtypes, ``to_dict`` round-trips, ``get`` has a
default, ``update_unuse`` applies the keys it knows and hands back the rest.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator

import torch

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
           "half": torch.float16, "fp32": torch.float32, "float32": torch.float32, "float": torch.float32,
           "fp64": torch.float64}


def get_dtype(name):
    if isinstance(name, torch.dtype) or name is None:
        return name
    if name not in _DTYPES:
        raise ValueError(f"unknown dtype {name!r}")
    return _DTYPES[name]


class ConfigNode:
    def __init__(self, d: Dict[str, Any]):
        for k, v in d.items():
            if k == "dtype" and isinstance(v, str):
                v = get_dtype(v)
            self.__dict__[k] = ConfigNode(v) if isinstance(v, dict) else v

    def to_dict(self) -> Dict[str, Any]:
        return {k: (v.to_dict() if isinstance(v, ConfigNode) else v) for k, v in self.__dict__.items()}

    def get(self, key: str, default=None):
        return self.__dict__.get(key, default)

    def __contains__(self, key):
        return key in self.__dict__

    def __iter__(self) -> Iterator[str]:
        return iter(self.__dict__)

    def items(self):
        return self.__dict__.items()

    def update_unuse(self, **kwargs) -> Dict[str, Any]:
        rest = {}
        for k, v in kwargs.items():
            if k in self.__dict__:
                setattr(self, k, v)
            else:
                rest[k] = v
        return rest

    def __repr__(self):
        return f"ConfigNode({self.to_dict()!r})"


def find_values(node, key: str):
    """Every value stored under ``key`` anywhere in the tree (used by the path checker)."""
    out = []
    if isinstance(node, ConfigNode):
        node = node.__dict__
    if isinstance(node, dict):
        for k, v in node.items():
            if k == key and not isinstance(v, (dict, ConfigNode)):
                out.append(v)
            out.extend(find_values(v, key))
    elif isinstance(node, (list, tuple)):
        for v in node:
            out.extend(find_values(v, key))
    return out
