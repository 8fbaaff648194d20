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


# ------------------------------------------------------------------------ environment queries, tensor layouts
def get_device_compute_capability() -> tuple:
    """(major, minor) of the current CUDA device; (0, 0) without one."""
    if not torch.cuda.is_available():
        return (0, 0)
    p = torch.cuda.get_device_properties(torch.cuda.current_device())
    return (p.major, p.minor)


def get_cudnn_version() -> tuple:
    """(major, minor, patch) of the cuDNN that PyTorch loaded (the attention kernels here do not use it)."""
    v = torch.backends.cudnn.version() or 0
    return (v // 10000, (v // 100) % 100, v % 100) if v >= 90000 else (v // 1000, (v // 100) % 10, v % 100)


def is_bf16_available(return_reason: bool = False):
    ok = (not torch.cuda.is_available()) or get_device_compute_capability() >= (8, 0)
    return (ok, "" if ok else "bf16 needs compute capability 8.0 or newer") if return_reason else ok


def torch_version() -> tuple:
    import re

    return tuple(int(x) for x in re.match(r"(\d+)\.(\d+)\.(\d+)", torch.__version__).groups())


def interleave_glu_tensor(tensor: torch.Tensor, interleave_size: int) -> torch.Tensor:
    """``[W_all, V_all]`` along dim 0 (gate rows, then linear rows) -> blocks of ``interleave_size`` rows alternating
    gate / linear: ``[W0:k, V0:k, Wk:2k, Vk:2k, ...]``.  Shape unchanged."""
    n = tensor.shape[0]
    if interleave_size <= 0 or n % (2 * interleave_size) != 0:
        raise ValueError(f"dimension 0 ({n}) must be a multiple of 2 * interleave_size ({interleave_size})")
    half = n // 2
    w, v = tensor[:half], tensor[half:]
    blocks = half // interleave_size
    rest = tensor.shape[1:]
    st = torch.stack([w.reshape(blocks, interleave_size, *rest), v.reshape(blocks, interleave_size, *rest)], dim=1)
    return st.reshape(n, *rest).contiguous()


def deinterleave_glu_tensor(tensor: torch.Tensor, interleave_size: int) -> torch.Tensor:
    """Inverse of :func:`interleave_glu_tensor`."""
    n = tensor.shape[0]
    if interleave_size <= 0 or n % (2 * interleave_size) != 0:
        raise ValueError(f"dimension 0 ({n}) must be a multiple of 2 * interleave_size ({interleave_size})")
    blocks = n // (2 * interleave_size)
    rest = tensor.shape[1:]
    t = tensor.reshape(blocks, 2, interleave_size, *rest)
    return torch.cat([t[:, 0].reshape(n // 2, *rest), t[:, 1].reshape(n // 2, *rest)], dim=0).contiguous()
from .helpers import *  # noqa: F401,F403,E402
