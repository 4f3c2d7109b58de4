"""Asynchronous CPU offload of checkpointed layer inputs.

With layer recomputation only each layer's input (hidden + residual stream) survives the forward pass; for long
micro-batches those inputs are still gigabytes. The offloader copies them to pinned host memory on a side stream right
after the layer consumed them and brings them back one layer ahead of the backward pass, so neither copy stalls compute:

    forward  layer i:   compute(i)      | side stream: D2H input(i)
    backward layer i:   recompute+bwd(i) | side stream: H2D input(i-1)

Pinned buffers are cached per (slot, shape) and reused across steps (allocation of pinned memory is slow).

Parity target: ``verl/utils/activation_offload.py`` (``AsyncDoubleBufferGroupOffloadHandler``, ``enable_activation_offloading``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

__all__ = ["ActivationOffloader", "OffloadHandle"]


@dataclass
class OffloadHandle:
    host: list                      # pinned host tensors (None entries stay None)
    device: Optional[list] = None   # filled by prefetch
    d2h_done: Optional[torch.cuda.Event] = None
    h2d_done: Optional[torch.cuda.Event] = None
    meta: list = field(default_factory=list)


class ActivationOffloader:
    def __init__(self, device):
        self.device = torch.device(device)
        self.enabled = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if self.enabled else None
        self._pinned: dict = {}
        self.bytes_offloaded = 0

    def _host_buffer(self, slot, j: int, t: torch.Tensor) -> torch.Tensor:
        key = (slot, j, tuple(t.shape), t.dtype)
        buf = self._pinned.get(key)
        if buf is None:
            buf = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            self._pinned[key] = buf
        return buf

    def offload(self, slot, tensors) -> OffloadHandle:
        """Start copying ``tensors`` (a tuple; entries may be None) to the host; the device copies may be dropped by the
        caller right away."""
        if not self.enabled:
            return OffloadHandle(host=list(tensors), device=list(tensors))
        cur = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        host = []
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            for j, t in enumerate(tensors):
                if t is None:
                    host.append(None)
                    continue
                buf = self._host_buffer(slot, j, t)
                buf.copy_(t, non_blocking=True)
                t.record_stream(self.stream)  # keep the device memory alive until the copy has run
                host.append(buf)
                self.bytes_offloaded += t.numel() * t.element_size()
            done = torch.cuda.Event()
            done.record(self.stream)
        return OffloadHandle(host=host, d2h_done=done)

    def prefetch(self, h: OffloadHandle) -> None:
        if not self.enabled or h.device is not None:
            return
        with torch.cuda.stream(self.stream):
            if h.d2h_done is not None:
                self.stream.wait_event(h.d2h_done)
            h.device = [None if b is None else b.to(self.device, non_blocking=True) for b in h.host]
            h.h2d_done = torch.cuda.Event()
            h.h2d_done.record(self.stream)

    def wait(self, h: OffloadHandle) -> tuple:
        """Device tensors of the handle, valid on the current stream."""
        if not self.enabled:
            return tuple(h.device)
        if h.device is None:
            self.prefetch(h)
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(h.h2d_done)
        for t in h.device:
            if t is not None:
                t.record_stream(cur)
        return tuple(h.device)
