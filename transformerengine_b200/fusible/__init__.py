"""Operation fuser: a ``Sequential`` of small operations that is pattern-matched into the fused
kernels of this library before it runs (reference: ``pytorch/ops/op.py:59,176,788``,
``pytorch/ops/fuser.py:53,400,751``, ``pytorch/ops/fused/*.py``).

Fusions applied (greedy, longest first):

* ``Norm, Linear, Activation, Linear``  -> one LayerNormMLP pass (norm+quantize, fc1, act+quantize, fc2)
* ``Norm, Linear``                       -> LayerNormLinear (norm output is written quantized)
* ``Linear, Activation``                 -> GEMM followed by the activation(+quantize) kernel
* ``AddExtraInput`` after a ``Linear``   -> residual add on the GEMM output

The fused modules share the ``Parameter`` objects of the basic operations, so state dicts and
optimizers only ever see the basic operations.
"""
from .ops import (FusibleOperation, BasicLinear, Bias, Linear, LayerNorm, RMSNorm, GELU, ReLU, SiLU, SwiGLU, GEGLU,
                  ReGLU, QGELU, SReLU, Quantize, Identity, Reshape, ConstantScale, Dropout, AddExtraInput,
                  MakeExtraOutput, AllReduce, AllGather, ReduceScatter, L2Normalization)
from .sequential import Sequential, fuse_operations

__all__ = ["FusibleOperation", "BasicLinear", "Bias", "Linear", "LayerNorm", "RMSNorm", "GELU", "ReLU", "SiLU",
           "SwiGLU", "GEGLU", "ReGLU", "QGELU", "SReLU", "Quantize", "Identity", "Reshape", "ConstantScale",
           "Dropout", "AddExtraInput", "MakeExtraOutput", "AllReduce", "AllGather", "ReduceScatter",
           "L2Normalization", "Sequential", "fuse_operations"]
