"""Small runtime utilities: NVTX ranges, device-side timers, environment flags
(reference: ``pytorch/utils.py`` nvtx helpers, ``common/util/logging.h``, env flags ``NVTE_*``)."""
from __future__ import annotations

import contextlib
import os
from typing import Dict, List

import torch

from .config import Config, get_config, override, reload_from_env, set_config  # noqa: F401,E402

_NVTX_ENABLED = get_config().nvtx


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a region (no-op unless ``TEB200_NVTX=1`` and CUDA is present)."""
    on = _NVTX_ENABLED and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def env_flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    return default if v is None else v.strip().lower() in ("1", "true", "yes", "on")


def env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class DeviceTimers:
    """Named CUDA-event timers: ``with timers("fwd"): ...`` then ``timers.summary()`` in ms."""

    def __init__(self):
        self._events: Dict[str, List] = {}

    @contextlib.contextmanager
    def __call__(self, name: str):
        if not torch.cuda.is_available():
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self._events.setdefault(name, []).append((a, b))

    def summary(self) -> Dict[str, float]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k, v in self._events.items()}

    def reset(self):
        self._events.clear()
