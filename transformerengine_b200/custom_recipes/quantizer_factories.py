"""Single-format factories: each returns the quantizer of one tensor role.

A factory is called once per quantizer slot with the slot's role -- ``"linear_input"``,
``"linear_weight"``, ``"linear_output"``, ``"linear_grad_output"`` or ``"linear_grad_input"`` (an
object with a ``tensor_type`` attribute of ``"input" | "weight" | "output" | "grad_output" |
"grad_input"`` is accepted too) -- and returns a quantizer, or ``None`` to keep that tensor in high
precision.  (Reference: ``pytorch/custom_recipes/quantizer_factories.py:35-140``.)
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from ..tensor import (Float8BlockQuantizer, Float8CurrentScalingQuantizer, IdentityQuantizer, MXFP8Quantizer,
                      NVFP4Quantizer)

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


def tensor_type(role: Any) -> str:
    """``"input" | "weight" | "output" | "grad_output" | "grad_input"`` of a role."""
    t = getattr(role, "tensor_type", role)
    t = str(t)
    return t[len("linear_"):] if t.startswith("linear_") else t


def is_backward(role: Any) -> bool:
    return tensor_type(role).startswith("grad")


def _skip(role: Any) -> bool:  # GEMM outputs stay in high precision unless a caller asks otherwise
    return tensor_type(role) in ("output", "grad_input")


def high_precision_factory(role: Any) -> Optional[Any]:
    return None


def identity_factory(role: Any):
    return None if _skip(role) else IdentityQuantizer()


def current_scaling_factory(role: Any, *, hybrid_format: bool = True, force_pow_2_scales: bool = False,
                            amax_epsilon: float = 0.0):
    if _skip(role):
        return None
    dtype = E5M2 if (hybrid_format and is_backward(role)) else E4M3
    return Float8CurrentScalingQuantizer(dtype, force_pow_2_scales=force_pow_2_scales, amax_epsilon=amax_epsilon)


def float8_block_scaling_factory(role: Any, *, force_pow_2_scales: bool = True, amax_epsilon: float = 0.0):
    """1x128 blocks for activations and gradients, 128x128 blocks for weights."""
    if _skip(role):
        return None
    dim = 2 if tensor_type(role) == "weight" else 1
    return Float8BlockQuantizer(E4M3, block_scaling_dim=dim, force_pow_2_scales=force_pow_2_scales,
                                amax_epsilon=amax_epsilon)


def mxfp8_factory(role: Any, *, hybrid_format: bool = False):
    if _skip(role):
        return None
    return MXFP8Quantizer(E5M2 if (hybrid_format and is_backward(role)) else E4M3)


def nvfp4_factory(role: Any, *, random_hadamard_transform: bool = True, stochastic_rounding: bool = True,
                  weight_2d: bool = True):
    """The NVFP4 training recipe: RHT on the columnwise copy of inputs and gradients, stochastic
    rounding on gradients, 16x16 blocks on weights."""
    if _skip(role):
        return None
    t = tensor_type(role)
    if t == "weight":
        return NVFP4Quantizer(with_2d_quantization=weight_2d)
    return NVFP4Quantizer(with_rht=random_hadamard_transform,
                          stochastic_rounding=stochastic_rounding and t == "grad_output")
