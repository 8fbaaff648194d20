"""Small helpers for looking at FP8 numerics by hand (reference: ``pytorch/numerics_debug.py``)."""
from __future__ import annotations

from typing import Tuple

import torch

_ENABLED = False
_FP8_MAX = {"E4M3": 448.0, "E5M2": 57344.0}


def debug(enabled: bool = True) -> None:
    """Switch the module-level debug flag (read by callers that want extra checks)."""
    global _ENABLED
    _ENABLED = enabled


def is_debug() -> bool:
    return _ENABLED


def fp8_tensor_statistics(tensor: torch.Tensor, fp8_format: str = "E4M3") -> Tuple[int, int]:
    """(underflows, overflows) of values that were cast to FP8 and back: entries that became zero
    and entries that sit at the format's largest magnitude."""
    fmt = fp8_format.upper()
    assert fmt in _FP8_MAX, "fp8_format must be 'E4M3' or 'E5M2'"
    t = tensor.float()
    return int((t == 0).sum().item()), int((t.abs() == _FP8_MAX[fmt]).sum().item())
