"""Asynchronous host prefetch + pinned staging + H2D on a side stream.

A background thread pulls collated batches, pins them, and (on CUDA) issues the host-to-device copies on
its own stream so that the copy of step i+1 overlaps the compute of step i; ``next()`` hands out device
batches after making the compute stream wait for the copy.  Reference: the ``Preloader`` of
mindspeed_mm/fsdp/data/dataloader/dataloader.py:165-256 (prefetch thread, H2D triggered after backward).
"""
from __future__ import annotations

import queue
import threading
from typing import Iterable, Optional

import torch

from .collate import pin_batch, to_device


class Preloader:
    def __init__(self, batches: Iterable[dict], device, depth: int = 2):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.q: "queue.Queue" = queue.Queue(maxsize=depth)
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self._src = batches
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        try:
            for b in self._src:
                if self._stop.is_set():
                    return
                if self.cuda:
                    b = pin_batch(b)
                    with torch.cuda.stream(self.stream):
                        d = to_device(b, self.device, non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(self.stream)
                    self.q.put((d, ev, b))
                else:
                    self.q.put((b, None, None))
            self.q.put(None)
        except BaseException as e:  # noqa: BLE001  (surface loader errors in the training thread)
            self.q.put(e)

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        item = self.q.get()
        if item is None:
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        d, ev, _host = item
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        return d

    def close(self):
        self._stop.set()
