"""Mixed-format factories: different formats for the forward and the backward pass, or for the two
directions of one tensor (reference: ``pytorch/custom_recipes/quantizer_factory_zoo.py:83-356``).

Which GEMM reads what: fprop reads the rowwise copies of input and weight; dgrad the rowwise
gradient and the columnwise weight; wgrad the columnwise gradient and the columnwise input.  A
tensor whose two directions feed GEMMs of different formats gets a ``HybridQuantizer``.
"""
from __future__ import annotations

from typing import Any

from ..tensor import HybridQuantizer, IdentityQuantizer, MXFP8Quantizer, NVFP4Quantizer
from .quantizer_factories import E4M3, E5M2, _skip, tensor_type


def mxfp8_fwd_nvfp4_bwd_factory(role: Any):
    """Forward GEMM in MXFP8, both backward GEMMs in NVFP4."""
    if _skip(role):
        return None
    t = tensor_type(role)
    if t == "grad_output":
        return NVFP4Quantizer(with_rht=True, stochastic_rounding=True)
    col = NVFP4Quantizer(with_rht=(t == "input"))
    return HybridQuantizer(rowwise_quantizer=MXFP8Quantizer(E4M3), columnwise_quantizer=col)


def high_precision_fwd_mxfp8_bwd_factory(role: Any):
    """Forward GEMM in high precision, backward GEMMs in MXFP8."""
    if _skip(role):
        return None
    if tensor_type(role) == "grad_output":
        return MXFP8Quantizer(E5M2)
    return HybridQuantizer(rowwise_quantizer=IdentityQuantizer(), columnwise_quantizer=MXFP8Quantizer(E4M3))


def mxfp8_fwd_high_precision_bwd_factory(role: Any):
    """Forward GEMM in MXFP8, backward GEMMs in high precision."""
    if _skip(role):
        return None
    if tensor_type(role) == "grad_output":
        return None
    return HybridQuantizer(rowwise_quantizer=MXFP8Quantizer(E4M3), columnwise_quantizer=IdentityQuantizer())


def nvfp4_1d_weight_factory(role: Any):
    """NVFP4 everywhere with 1-D (1x16) weight blocks whose columnwise copy is quantized from the
    dequantized rowwise copy, so that dgrad sees the values fprop used (double quantization)."""
    if _skip(role):
        return None
    t = tensor_type(role)
    if t == "weight":
        return HybridQuantizer(rowwise_quantizer=NVFP4Quantizer(), columnwise_quantizer=NVFP4Quantizer(),
                               columnwise_source="rowwise_dequantized")
    return NVFP4Quantizer(with_rht=True, stochastic_rounding=t == "grad_output")
