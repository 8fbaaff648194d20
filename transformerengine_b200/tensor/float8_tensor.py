"""Per-tensor scaled FP8 tensors and quantizers (the reference's module name ``pytorch/tensor/float8_tensor.py``; the classes live in ``tensor/float8.py``)."""
from .float8 import *  # noqa: F401,F403
from .float8 import Float8CurrentScalingQuantizer, Float8Quantizer, Float8Tensor, Float8TensorStorage, _make_float8_tensor_in_reduce_ex  # noqa: F401
