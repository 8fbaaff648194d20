"""MXFP8 tensors and quantizer (the reference's module name ``pytorch/tensor/mxfp8_tensor.py``; the classes live in ``tensor/mxfp8.py``)."""
from .mxfp8 import *  # noqa: F401,F403
from .mxfp8 import MXFP8Quantizer, MXFP8Tensor, MXFP8TensorStorage, _make_mxfp8_tensor_in_reduce_ex  # noqa: F401
