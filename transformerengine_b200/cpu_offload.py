"""Activation offloading to pinned host memory (reference: ``pytorch/cpu_offload.py:90,228,495,692``).

``get_cpu_offload_context`` returns a context manager and a synchronisation function::

    ctx, sync = get_cpu_offload_context(enabled=True, num_layers=4, model_layers=32)
    for layer in layers:
        with ctx:
            x = layer(x)
        x = sync(x)

Tensors saved for backward inside the context of the first ``num_layers`` layers are copied to
pinned host buffers on a side stream (device-to-host overlaps the next layer's compute) and
copied back, one layer ahead, when the backward pass reaches them.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch


class _OffloadHandler:
    def __init__(self, num_layers: int, model_layers: int, min_numel: int = 1 << 16):
        self.num_offload, self.model_layers, self.min_numel = num_layers, model_layers, min_numel
        self.layer = 0
        self.cuda = torch.cuda.is_available()
        self.d2h = torch.cuda.Stream() if self.cuda else None
        self.h2d = torch.cuda.Stream() if self.cuda else None
        self.store: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.device, Optional[torch.cuda.Event]]] = {}
        self.counter = 0
        self.bytes_offloaded = 0

    def should_offload(self, t: torch.Tensor) -> bool:
        return (self.layer < self.num_offload and isinstance(t, torch.Tensor) and t.numel() >= self.min_numel
                and not isinstance(t, torch.nn.Parameter) and (t.is_cuda or not self.cuda))

    def pack(self, t):
        if not self.should_offload(t):
            return t
        key = (self.layer, self.counter)
        self.counter += 1
        if self.cuda and t.is_cuda:
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            self.d2h.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.d2h):
                host.copy_(t, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.d2h)
            t.record_stream(self.d2h)
        else:
            host, ev = t.detach().clone(), None
        self.bytes_offloaded += t.numel() * t.element_size()
        self.store[key] = (host, t.device, ev)
        return ("__offloaded__", key)

    def unpack(self, obj):
        if not (isinstance(obj, tuple) and len(obj) == 2 and obj[0] == "__offloaded__"):
            return obj
        host, dev, ev = self.store.pop(obj[1])
        if self.cuda and dev.type == "cuda":
            if ev is not None:
                self.h2d.wait_event(ev)
            with torch.cuda.stream(self.h2d):
                out = host.to(dev, non_blocking=True)
            torch.cuda.current_stream().wait_stream(self.h2d)
            out.record_stream(torch.cuda.current_stream())
            return out
        return host

    def next_layer(self):
        self.layer += 1
        if self.layer >= self.model_layers:
            self.layer = 0


class _OffloadContext:
    def __init__(self, handler: Optional[_OffloadHandler]):
        self.handler = handler
        self._hooks = None

    def __enter__(self):
        if self.handler is not None:
            self._hooks = torch.autograd.graph.saved_tensors_hooks(self.handler.pack, self.handler.unpack)
            self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        if self._hooks is not None:
            self._hooks.__exit__(*exc)
            self._hooks = None
        return False


def get_cpu_offload_context(enabled: bool = False, num_layers: Optional[int] = 1, model_layers: int = 1,
                            offload_activations: bool = True, offload_weights: bool = False,
                            double_buffering: bool = False, manual_synchronization: bool = False,
                            retain_pinned_cpu_buffers: bool = False, offload_stream=None):
    """Returns ``(context, sync_function)``; ``sync_function(tensor)`` marks the end of a layer."""
    if not enabled or not offload_activations:
        return _OffloadContext(None), (lambda t: t)
    handler = _OffloadHandler(num_layers or 0, model_layers)

    def sync(t):
        handler.next_layer()
        return t

    ctx = _OffloadContext(handler)
    ctx.handler = handler
    return ctx, sync
