"""Memory features applied around modules: asynchronous activation offload and chunked micro-batches.

* ``ActivationOffload`` - ``saved_tensors_hooks`` that move tensors saved for backward to pinned host memory on
  a D2H stream during forward and bring them back on an H2D stream just before they are needed (one unit of
  look-ahead), keeping only small tensors on the device.  Reference: mindspeed_mm/fsdp/features/memory/
  async_offload.py:67-331.  On a B200 (180 GB) this is for long-sequence DiT runs; units under full recompute
  only save their inputs, which is exactly what gets offloaded.
* ``chunk_mbs`` - run a module on slices of the batch dimension and concatenate the results, bounding the
  activation peak of that module (mindspeed_mm/fsdp/features/communication/chunk_mbs.py:40-111).
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class ActivationOffload:
    def __init__(self, device=None, min_bytes: int = 1 << 20, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.min_bytes = min_bytes
        self.device = device
        self.d2h = torch.cuda.Stream() if self.enabled else None
        self.h2d = torch.cuda.Stream() if self.enabled else None
        self.bytes_offloaded = 0

    def _pack(self, t: torch.Tensor):
        if (not self.enabled) or (not t.is_cuda) or t.numel() * t.element_size() < self.min_bytes or \
                isinstance(t, torch.nn.Parameter):
            return ("keep", t)
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        self.d2h.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.d2h):
            host.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.d2h)
        t.record_stream(self.d2h)
        self.bytes_offloaded += t.numel() * t.element_size()
        return ("host", host, ev, t.device)

    def _unpack(self, packed):
        if packed[0] == "keep":
            return packed[1]
        _, host, ev, dev = packed
        with torch.cuda.stream(self.h2d):
            self.h2d.wait_event(ev)
            out = host.to(dev, non_blocking=True)
        torch.cuda.current_stream().wait_stream(self.h2d)
        return out

    def __enter__(self):
        self._ctx = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._ctx.__enter__()
        return self

    def __exit__(self, *a):
        return self._ctx.__exit__(*a)

    def wrap(self, module: torch.nn.Module) -> torch.nn.Module:
        """Run ``module.forward`` under the hooks from now on."""
        fwd = module.forward

        def forward(*args, **kw):
            with self:
                return fwd(*args, **kw)
        module.forward = forward
        return module


def chunk_mbs(fn: Callable, chunk: int, batch_dim: int = 0, arg_indexes: Sequence[int] = (0,), kwarg_names: Sequence[str] = ()):
    """Wrap ``fn`` so that the listed tensor arguments are split into slices of ``chunk`` along ``batch_dim``."""
    def wrapped(*args, **kwargs):
        ref = args[arg_indexes[0]]
        n = ref.shape[batch_dim]
        if n <= chunk:
            return fn(*args, **kwargs)
        outs = []
        for s in range(0, n, chunk):
            a = list(args)
            for i in arg_indexes:
                a[i] = args[i].narrow(batch_dim, s, min(chunk, n - s))
            kw = dict(kwargs)
            for k in kwarg_names:
                if isinstance(kw.get(k), torch.Tensor) and kw[k].dim() > batch_dim and kw[k].shape[batch_dim] == n:
                    kw[k] = kw[k].narrow(batch_dim, s, min(chunk, n - s))
            outs.append(fn(*a, **kw))
        if isinstance(outs[0], tuple):
            return tuple(torch.cat([o[j] for o in outs], dim=batch_dim) for j in range(len(outs[0])))
        return torch.cat(outs, dim=batch_dim)
    return wrapped
