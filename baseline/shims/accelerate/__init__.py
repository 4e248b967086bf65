"""Stand-in for the one `accelerate` symbol the reference's model hub imports."""
from contextlib import contextmanager

import torch
import torch.nn as nn

__version__ = "0.0.0+standin"


@contextmanager
def init_empty_weights(include_buffers: bool = False):
    """Inside the context every parameter a module registers lands on the meta device (no storage).
    Buffers keep their real device unless ``include_buffers``."""
    old_register_parameter = nn.Module.register_parameter
    old_register_buffer = nn.Module.register_buffer
    meta = torch.device("meta")

    def register_parameter(module, name, param):
        old_register_parameter(module, name, param)
        if param is not None:
            p = module._parameters[name]
            cls = type(p)
            kwargs = dict(p.__dict__)
            kwargs["requires_grad"] = p.requires_grad
            module._parameters[name] = cls(p.to(meta), **kwargs)

    def register_buffer(module, name, tensor, persistent=True):
        old_register_buffer(module, name, tensor, persistent=persistent)
        if tensor is not None:
            module._buffers[name] = module._buffers[name].to(meta)

    nn.Module.register_parameter = register_parameter
    if include_buffers:
        nn.Module.register_buffer = register_buffer
    try:
        yield
    finally:
        nn.Module.register_parameter = old_register_parameter
        nn.Module.register_buffer = old_register_buffer
