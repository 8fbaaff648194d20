"""``recipe.fp8_dpa`` / ``recipe.fp8_mha`` and ``fp8_output`` of the core attention, as FP8 rounding AROUND the 16-bit
attention kernels.

The reference hands FP8 Q, K, V to cuDNN's FP8 attention (``attention/dot_product_attention/backends.py``,
``FusedAttnFunc`` with ``fp8=True``): the tensors entering and leaving the attention are FP8, the products accumulate
in fp32.  The tcgen05 attention kernels here take fp16 / bf16, so FP8 attention is reproduced at the tensor boundaries:

* forward: Q, K and V are rounded to the recipe's forward format (per-tensor scale from the tensor's own amax; 1 x 32
  block scales under an MXFP8 recipe) and read back in the input dtype; with ``fp8_mha`` / ``fp8_output`` the
  attention output is rounded the same way;
* backward (unless ``NVTE_FP8_DPA_BWD=0`` or ``bf16_backward``): dO and dQ, dK, dV are rounded to the recipe's
  gradient format.

What this does NOT reproduce is the rounding of the probabilities P and of dP inside the kernel, and it saves no
time or memory: it exists so that models configured for FP8 attention run, with the boundary numerics of that
configuration, and so that the accuracy effect of FP8 Q/K/V/O can be studied.  Delayed-scaling recipes use the
current amax here (no history for the attention tensors).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..common.recipe import Format


def _dtypes(recipe) -> Tuple[torch.dtype, torch.dtype]:
    fmt = getattr(recipe, "fp8_format", Format.HYBRID)
    fwd = torch.float8_e5m2 if fmt == Format.E5M2 else torch.float8_e4m3fn
    bwd = torch.float8_e4m3fn if fmt == Format.E4M3 else torch.float8_e5m2
    return fwd, bwd


def _round_trip(x: torch.Tensor, fp8_dtype: torch.dtype, mx: bool) -> torch.Tensor:
    """``x`` rounded to FP8 and read back in its own dtype (the head dim is the row of a 2-D view)."""
    from ..tensor.float8 import Float8CurrentScalingQuantizer
    from ..tensor.mxfp8 import MXFP8Quantizer
    if x.numel() == 0:
        return x
    flat = x.reshape(-1, x.shape[-1])
    if not flat.is_contiguous():
        flat = flat.contiguous()
    q = None
    if mx:
        q = MXFP8Quantizer(fp8_dtype, rowwise=True, columnwise=False)
        if not q.is_quantizable(flat):
            q = None        # ragged shapes take the per-tensor scale
    if q is None:
        q = Float8CurrentScalingQuantizer(fp8_dtype, device=x.device, rowwise=True, columnwise=False)
    return q(flat.detach()).dequantize(dtype=x.dtype).reshape(x.shape)


class _Fp8Boundary(torch.autograd.Function):
    """Round the forward value to ``fwd`` (None: pass through) and the gradient to ``bwd`` (None: pass through)."""

    @staticmethod
    def forward(ctx, x, fwd: Optional[torch.dtype], bwd: Optional[torch.dtype], mx: bool):  # type: ignore[override]
        ctx.bwd, ctx.mx = bwd, mx
        return x.clone() if fwd is None else _round_trip(x, fwd, mx)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return (g if ctx.bwd is None else _round_trip(g, ctx.bwd, ctx.mx)), None, None, None


class Fp8AttentionBoundary:
    """What to round around one attention call; built from the active recipe by ``plan``."""

    def __init__(self, fwd: torch.dtype, bwd: Optional[torch.dtype], mx: bool, quantize_output: bool):
        self.fwd, self.bwd, self.mx, self.quantize_output = fwd, bwd, mx, quantize_output

    def inputs(self, *tensors):
        return tuple(None if t is None else _Fp8Boundary.apply(t, self.fwd, self.bwd, self.mx) for t in tensors)

    def output(self, o: torch.Tensor) -> torch.Tensor:
        if not self.quantize_output and self.bwd is None:
            return o
        return _Fp8Boundary.apply(o, self.fwd if self.quantize_output else None, self.bwd, self.mx)


def plan(fp8_output: bool = False, bf16_backward: bool = False) -> Optional[Fp8AttentionBoundary]:
    """The boundary rounding the active autocast asks for, or None (no autocast, or a recipe without ``fp8_dpa`` /
    ``fp8_mha`` and no ``fp8_output``)."""
    from ..quantization import FP8GlobalStateManager
    from ..utils.config import get_config
    if not FP8GlobalStateManager.is_fp8_enabled():
        if fp8_output:
            raise ValueError("fp8_output=True needs an enabled autocast")
        return None
    rec = FP8GlobalStateManager.get_fp8_recipe()
    dpa, mha = bool(getattr(rec, "fp8_dpa", False)), bool(getattr(rec, "fp8_mha", False))
    if not (dpa or mha or fp8_output):
        return None
    fwd, bwd = _dtypes(rec)
    if bf16_backward or not get_config().fp8_dpa_bwd:
        bwd = None
    mx = bool(getattr(rec, "mxfp8", lambda: False)())
    return Fp8AttentionBoundary(fwd, bwd, mx, quantize_output=mha or fp8_output)
