"""Reference GEMM on quantized operands: dequantize, multiply in fp32, cast.  The oracle for
custom quantizers that the tensor-core kernels do not know (reference: ``pytorch/custom_recipes/gemm.py:35``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..tensor.base import QuantizedTensorStorage


def _values(t, usage: str) -> torch.Tensor:
    from ..tensor.hybrid import HybridQuantizedTensorStorage

    if isinstance(t, HybridQuantizedTensorStorage):
        child = t._rowwise if usage == "rowwise" else t._columnwise
        t = child if child is not None else t
    if isinstance(t, QuantizedTensorStorage):
        return t.dequantize(dtype=torch.float32)
    return t.float()


def custom_gemm(A, B, *, layout: str = "TN", out_dtype: Optional[torch.dtype] = None, bias: Optional[torch.Tensor] = None,
                accumulate: bool = False, out: Optional[torch.Tensor] = None, alpha: float = 1.0) -> torch.Tensor:
    """``layout`` as in ``general_gemm``: "TN" ``out = B @ A^T`` (fprop: A weight, B input), "NN"
    ``out = B @ A`` (dgrad: A weight, B grad), "NT" ``out = B^T @ A`` (wgrad: A input, B grad)."""
    assert layout in ("TN", "NN", "NT")
    if layout == "TN":
        a, b = _values(A, "rowwise"), _values(B, "rowwise")
        res = b.reshape(-1, b.shape[-1]) @ a.reshape(-1, a.shape[-1]).t()
        lead = tuple(b.shape[:-1])
    elif layout == "NN":
        a, b = _values(A, "columnwise"), _values(B, "rowwise")
        res = b.reshape(-1, b.shape[-1]) @ a.reshape(-1, a.shape[-1])
        lead = tuple(b.shape[:-1])
    else:
        a, b = _values(A, "columnwise"), _values(B, "columnwise")
        res = b.reshape(-1, b.shape[-1]).t() @ a.reshape(-1, a.shape[-1])
        lead = None
    res = res * alpha
    if bias is not None:
        res = res + bias.float()
    if lead is not None:
        res = res.reshape(*lead, res.shape[-1])
    if out is not None:
        out.copy_((out.float() + res if accumulate else res).to(out.dtype))
        return out
    return res.to(out_dtype or torch.float32)
