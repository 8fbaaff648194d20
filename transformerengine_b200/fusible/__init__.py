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
from .sequential import (Sequential, fuse_operations, register_backward_fusion, register_forward_backward_fusion,
                         register_forward_fusion, unregister_fusion)

BasicOperation = FusibleOperation     # the reference's names of the operation base classes
FusedOperation = FusibleOperation
# The reference has one fused class per pattern and per pass; here one chain module covers the linear patterns in
# both passes and one module the residual-fork + norm pattern.  The reference's class names point at them.
ForwardLinearBiasActivation = ForwardLinearBiasAdd = ForwardLinearScaleAdd = LinearChain
BackwardActivationBias = BackwardLinearAdd = BackwardLinearScale = LinearChain
BackwardAddRMSNorm = ForkNorm

__all__ = ["FusibleOperation", "BasicLinear", "Bias", "Linear", "LayerNorm", "RMSNorm", "GELU", "ReLU", "SiLU",
           "SwiGLU", "GEGLU", "ReGLU", "QGELU", "SReLU", "Quantize", "Identity", "Reshape", "ConstantScale",
           "Dropout", "AddExtraInput", "MakeExtraOutput", "AllReduce", "AllGather", "ReduceScatter",
           "L2Normalization", "GroupedLinear", "ScaledSwiGLU", "GLU", "QGEGLU", "SReGLU", "ClampedSwiGLU", "SiTUGLU",
           "ScaledSReLU", "ScaledClampedQGeGLU", "ScaledSiTUGLU", "Sequential", "fuse_operations", "register_forward_fusion", "register_backward_fusion",
           "register_forward_backward_fusion", "unregister_fusion", "BasicOperation", "FusedOperation", "LinearChain", "ForkNorm",
           "GroupedMLP"]
