"""Activation offloading to pinned host memory (reference: ``pytorch/cpu_offload.py:90,228,495,692``).

``get_cpu_offload_context`` returns a context manager and a synchronisation function::

    ctx, sync = get_cpu_offload_context(enabled=True, num_layers=4, model_layers=32)
    for layer in layers:
        with ctx:
            x = layer(x)
        x = sync(x)

Tensors saved for backward inside the context of the first ``num_layers`` layers are copied to pinned
host buffers on a side stream (the device-to-host copy overlaps the next layer's compute).  In the
backward pass the first use of a tensor of layer L reloads ALL tensors of layer L and, one layer ahead,
those of layer L - 1, so the host-to-device copies overlap the backward of layer L.

Options (all implemented):

* ``retain_pinned_cpu_buffers``: the pinned host buffers go back to a pool (by shape and dtype) once their
  reload has been issued and are reused by later offloads (``cudaHostAlloc`` per tensor and step is slow).
* ``double_buffering``: reloaded tensors land in two sets of device buffers that alternate by layer parity
  and are reused across iterations, instead of freshly allocated memory: the device footprint of the
  reloads is fixed (what a captured CUDA graph or a tight memory plan needs).  Assumes one forward /
  backward pass in flight at a time.
* ``manual_synchronization``: a third return value controls the copies by hand
  (``start_offload_layer`` / ``release_activation_forward_gpu_memory`` / ``start_reload_layer``); the
  hooks then only record and hand out tensors.
* ``offload_stream``: the stream the copies run on (default: two private streams).
* ``offload_weights``: not supported (the reference deprecated it); a warning is issued and it is ignored.
"""
from __future__ import annotations

import warnings
from typing import Dict, List, Optional, Tuple

import torch

_TAG = "__offloaded__"


class _Entry:
    __slots__ = ("host", "device", "event", "shape", "dtype", "src", "gpu", "gpu_event", "pos", "served")

    def __init__(self, pos):
        self.host = None       # pinned host copy (CPU runs: a detached clone)
        self.device = None
        self.event = None      # device-to-host copy finished
        self.shape = self.dtype = None
        self.src = None        # the device tensor until its copy has been issued (manual mode)
        self.gpu = None        # reloaded device tensor
        self.gpu_event = None  # host-to-device copy finished
        self.pos = pos
        self.served = False    # handed to the backward pass at least once


def mark_not_offload(*tensors) -> None:
    """Keep these tensors on the device even when they are saved inside an offload context (tensors that the
    backward pass needs first, or that are shared with other layers)."""
    for t in tensors:
        if isinstance(t, torch.Tensor):
            t._te_do_not_offload = True
        elif t is not None and hasattr(t, "get_data_tensors"):
            for d in t.get_data_tensors():
                if d is not None:
                    d._te_do_not_offload = True


_ACTIVE_CONTEXTS = [0]       # offload contexts currently entered


def is_cpu_offload_enabled() -> bool:
    """True inside an active offload context (modules use it to decide whether saved tensors may leave the GPU)."""
    return _ACTIVE_CONTEXTS[0] > 0


def mark_activation_offload(*tensors) -> None:
    """Mark tensors as activations that MAY be offloaded (clears a ``mark_not_offload`` mark).  Every tensor saved
    inside an offload context is a candidate already, so this only matters after ``mark_not_offload``."""
    for t in tensors:
        if isinstance(t, torch.Tensor):
            t._te_do_not_offload = False
        elif t is not None and hasattr(t, "get_data_tensors"):
            for d in t.get_data_tensors():
                if d is not None:
                    d._te_do_not_offload = False


def start_offload(*tensors, offload_base_tensor: bool = False) -> None:
    """Mark the point on the current stream where ``tensors`` are fully computed: their device-to-host copy, issued
    when they are saved for backward, waits for this point and not for later work on the stream.
    ``offload_base_tensor`` is accepted; views are offloaded as the tensors they are (each saved view is copied on
    its own)."""
    if not torch.cuda.is_available():
        return
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream())
    for t in tensors:
        parts = [t] if isinstance(t, torch.Tensor) else (
            [d for d in t.get_data_tensors() if d is not None] if (t is not None and hasattr(t, "get_data_tensors")) else [])
        for p in parts:
            p._te_ready_event = ev


class _OffloadHandler:
    def __init__(self, num_layers: int, model_layers: int, min_numel: int = 1 << 16, *, retain_pinned: bool = False,
                 double_buffering: bool = False, manual: bool = False, stream=None):
        self.num_offload, self.model_layers, self.min_numel = num_layers, model_layers, min_numel
        self.retain_pinned, self.double_buffering, self.manual = retain_pinned, double_buffering, manual
        self.layer = 0
        self.iteration = 0     # forward passes started so far: entries are keyed by (iteration, layer)
        self.cuda = torch.cuda.is_available()
        self.d2h = (stream or torch.cuda.Stream()) if self.cuda else None
        self.h2d = (stream or torch.cuda.Stream()) if self.cuda else None
        self.layers: Dict[Tuple[int, int], List[_Entry]] = {}   # (iteration, layer) -> entries in saving order
        self.reload_started: Dict[Tuple[int, int], bool] = {}
        self._pinned: Dict[tuple, list] = {}           # retained host buffers: (shape, dtype) -> [(tensor, last reader)]
        self._dbuf: Dict[tuple, torch.Tensor] = {}     # double buffers on the device
        self.bytes_offloaded = 0
        self.host_allocations = 0                      # pinned buffers created (stays flat with retain_pinned)

    # kept for introspection by tests: no entries left once the backward pass has consumed everything
    @property
    def store(self) -> dict:
        return {(k, e.pos): e for k, es in self.layers.items() for e in es}

    def should_offload(self, t) -> bool:
        return (self.layer < self.num_offload and isinstance(t, torch.Tensor) and t.numel() >= self.min_numel
                and not isinstance(t, torch.nn.Parameter) and (t.is_cuda or not self.cuda)
                and not getattr(t, "_te_do_not_offload", False))

    # ------------------------------------------------------------------ device -> host
    def _host_buffer(self, t: torch.Tensor) -> torch.Tensor:
        free = self._pinned.get((tuple(t.shape), t.dtype)) if self.retain_pinned else None
        if free:
            host, last_read = free.pop()
            if last_read is not None:
                self.d2h.wait_event(last_read)   # the reload that last read this buffer
            return host
        self.host_allocations += 1
        return torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)

    def _issue_offload(self, e: _Entry) -> None:
        t = e.src
        if t is None:
            return
        if self.cuda and t.is_cuda:
            e.host = self._host_buffer(t)
            ready = getattr(t, "_te_ready_event", None)
            if ready is not None:
                self.d2h.wait_event(ready)         # start_offload: the producer finished here, later work need not
            else:
                self.d2h.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.d2h):
                e.host.copy_(t, non_blocking=True)
                e.event = torch.cuda.Event()
                e.event.record(self.d2h)
            t.record_stream(self.d2h)
        else:
            e.host, e.event = t.detach().clone(), None
        e.src = None

    def pack(self, t):
        if not self.should_offload(t):
            return t
        key = (self.iteration, self.layer)
        entries = self.layers.setdefault(key, [])
        e = _Entry(len(entries))
        e.device, e.shape, e.dtype, e.src = t.device, tuple(t.shape), t.dtype, t
        entries.append(e)
        self.bytes_offloaded += t.numel() * t.element_size()
        if not self.manual:
            self._issue_offload(e)
        return (_TAG, key, e.pos)

    # ------------------------------------------------------------------ host -> device
    def _device_buffer(self, layer: int, e: _Entry) -> Optional[torch.Tensor]:
        if not self.double_buffering:
            return None
        key = (layer & 1, e.pos, e.shape, e.dtype)
        buf = self._dbuf.get(key)
        if buf is None:
            buf = self._dbuf[key] = torch.empty(e.shape, dtype=e.dtype, device=e.device)
        return buf

    def start_reload(self, key: Tuple[int, int]) -> None:
        """Issue the host-to-device copies of every tensor of layer ``key = (iteration, layer)`` (once)."""
        if self.reload_started.get(key) or key not in self.layers:
            return
        self.reload_started[key] = True
        layer = key[1]
        for e in self.layers[key]:
            if e.src is not None:       # manual mode, never offloaded: the device tensor is still there
                e.gpu, e.src = e.src, None
                continue
            if e.host is None or e.gpu is not None:
                continue
            if self.cuda and e.device.type == "cuda":
                if e.event is not None:
                    self.h2d.wait_event(e.event)
                if self.double_buffering:
                    # the buffer of this parity was last read by the backward of layer + 2
                    self.h2d.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.h2d):
                    dst = self._device_buffer(layer, e)
                    if dst is None:
                        e.gpu = e.host.to(e.device, non_blocking=True)
                    else:
                        dst.copy_(e.host, non_blocking=True)
                        e.gpu = dst
                    e.gpu_event = torch.cuda.Event()
                    e.gpu_event.record(self.h2d)
                if self.retain_pinned:
                    self._pinned.setdefault((e.shape, e.dtype), []).append((e.host, e.gpu_event))
            else:
                e.gpu = e.host
            e.host = None

    def unpack(self, obj):
        if not (isinstance(obj, tuple) and len(obj) == 3 and obj[0] == _TAG):
            return obj
        _, key, pos = obj
        if not self.manual:
            self.start_reload(key)
            self.start_reload((key[0], key[1] - 1))   # one layer ahead: overlaps this layer's backward
        e = self.layers[key][pos]
        if e.gpu is None:                  # manual mode without an explicit reload: do it now
            self.start_reload(key)
        out = e.gpu
        if e.gpu_event is not None:
            torch.cuda.current_stream().wait_event(e.gpu_event)
            out.record_stream(torch.cuda.current_stream())
            e.gpu_event = None
        e.served = True
        if all(x.served for x in self.layers[key]):
            # every tensor of the layer has gone to the backward pass: drop the bookkeeping (and with it the
            # handler's references to the reloaded tensors)
            del self.layers[key]
            self.reload_started.pop(key, None)
        return out

    def next_layer(self):
        self.layer += 1
        if self.layer >= self.model_layers:
            self.layer = 0
            self.iteration += 1


class ManualOffloadSynchronizer:
    """Hand control over the copies (``manual_synchronization=True``).  Layer numbers count the ``sync`` calls
    of the forward pass, starting at 0; they refer to the most recent forward pass that saved tensors for that
    layer.  (Reference: ``pytorch/cpu_offload.py`` ``ManualOffloadSynchronizer``.)"""

    def __init__(self, handler: _OffloadHandler):
        self._h = handler

    def _key(self, layer: int):
        keys = [k for k in self._h.layers if k[1] == layer]
        return max(keys) if keys else (self._h.iteration, layer)

    def start_offload_layer(self, layer: int) -> None:
        """Start copying the saved tensors of ``layer`` to the host."""
        for e in self._h.layers.get(self._key(layer), []):
            self._h._issue_offload(e)

    def release_activation_forward_gpu_memory(self, layer: int) -> None:
        """Make the current stream wait for the copies of ``layer``: after this point its device tensors are
        released as soon as their last reference goes away."""
        if not self._h.cuda:
            return
        for e in self._h.layers.get(self._key(layer), []):
            if e.event is not None:
                torch.cuda.current_stream().wait_event(e.event)

    def start_reload_layer(self, layer: int) -> None:
        """Start copying the tensors of ``layer`` back to the device."""
        self._h.start_reload(self._key(layer))


class _OffloadContext:
    def __init__(self, handler: Optional[_OffloadHandler]):
        self.handler = handler
        self._hooks = None

    def __enter__(self):
        if self.handler is not None:
            self._hooks = torch.autograd.graph.saved_tensors_hooks(self.handler.pack, self.handler.unpack)
            self._hooks.__enter__()
            _ACTIVE_CONTEXTS[0] += 1
        return self

    def __exit__(self, *exc):
        if self._hooks is not None:
            self._hooks.__exit__(*exc)
            self._hooks = None
            _ACTIVE_CONTEXTS[0] -= 1
        return False


def get_cpu_offload_context(enabled: bool = False, num_layers: Optional[int] = 1, model_layers: int = 1,
                            offload_activations: bool = True, offload_weights: bool = False,
                            double_buffering: bool = False, manual_synchronization: bool = False,
                            retain_pinned_cpu_buffers: bool = False, offload_stream=None):
    """Returns ``(context, sync_function)``, or ``(context, sync_function, ManualOffloadSynchronizer)`` with
    ``manual_synchronization=True``; ``sync_function(tensor)`` marks the end of a layer."""
    if offload_weights:
        warnings.warn("offload_weights is not supported (the reference deprecated it): only activations are offloaded",
                      stacklevel=2)
    if not enabled or not offload_activations:
        ctx = _OffloadContext(None)
        return (ctx, (lambda t: t), None) if manual_synchronization else (ctx, (lambda t: t))
    handler = _OffloadHandler(num_layers or 0, model_layers, retain_pinned=retain_pinned_cpu_buffers,
                              double_buffering=double_buffering, manual=manual_synchronization, stream=offload_stream)

    def sync(t):
        handler.next_layer()
        return t

    ctx = _OffloadContext(handler)
    if manual_synchronization:
        return ctx, sync, ManualOffloadSynchronizer(handler)
    return ctx, sync
