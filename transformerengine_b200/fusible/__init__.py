"""Operation fuser: a ``Sequential`` of small operations that is pattern-matched into the fused
kernels of this library before it runs (reference: ``pytorch/ops/op.py:59,176,788``,
``pytorch/ops/fuser.py:53,400,751``, ``pytorch/ops/fused/*.py``).

Fusions applied (greedy, longest first):

* ``Norm, Linear, Activation, Linear``  -> one LayerNormMLP pass (norm+quantize, fc1, act+quantize, fc2)
* ``Norm, Linear``                       -> LayerNormLinear (norm output is written quantized)
* ``Linear (, Bias) (, Activation) (, AddExtraInput)`` and ``Linear, ConstantScale (, AddExtraInput)``
                                         -> ``fused.LinearChain``: scale and bias in the GEMM epilogue; in the
                                            backward ONE kernel yields the activation gradient, the bias
                                            gradient and the quantized operands of dgrad / wgrad
* ``MakeExtraOutput, Norm``              -> ``fused.ForkNorm``: the norm backward kernel adds the gradient of
                                            the forked (residual) branch
* tensor-parallel ``Linear`` operations run the collective inside the GEMM kernel once ``initialize_ub`` was
  called (the reference's Userbuffers forward / backward linear fusions)

The fused modules share the ``Parameter`` objects of the basic operations, so state dicts and
optimizers only ever see the basic operations.
"""
from .ops import (FusibleOperation, BasicLinear, Bias, Linear, LayerNorm, RMSNorm, GELU, ReLU, SiLU, SwiGLU, GEGLU,
                  ReGLU, QGELU, SReLU, Quantize, Identity, Reshape, ConstantScale, Dropout, AddExtraInput,
                  MakeExtraOutput, AllReduce, AllGather, ReduceScatter, L2Normalization, GroupedLinear,
                  ScaledSwiGLU, GLU, QGEGLU, SReGLU, ClampedSwiGLU, SiTUGLU, ScaledSReLU, ScaledClampedQGeGLU,
                  ScaledSiTUGLU)
from .fused import ForkNorm, GroupedMLP, LinearChain
from .sequential import Sequential, fuse_operations

__all__ = ["FusibleOperation", "BasicLinear", "Bias", "Linear", "LayerNorm", "RMSNorm", "GELU", "ReLU", "SiLU",
           "SwiGLU", "GEGLU", "ReGLU", "QGELU", "SReLU", "Quantize", "Identity", "Reshape", "ConstantScale",
           "Dropout", "AddExtraInput", "MakeExtraOutput", "AllReduce", "AllGather", "ReduceScatter",
           "L2Normalization", "GroupedLinear", "ScaledSwiGLU", "GLU", "QGEGLU", "SReGLU", "ClampedSwiGLU", "SiTUGLU",
           "ScaledSReLU", "ScaledClampedQGeGLU", "ScaledSiTUGLU", "Sequential", "fuse_operations", "LinearChain", "ForkNorm",
           "GroupedMLP"]
