"""NVFP4 tensors and quantizer (the reference's module name ``pytorch/tensor/nvfp4_tensor.py``; the classes live in ``tensor/nvfp4.py``)."""
from .nvfp4 import *  # noqa: F401,F403
from .nvfp4 import NVFP4Quantizer, NVFP4Tensor, NVFP4TensorStorage, _make_nvfp4_tensor_in_reduce_ex  # noqa: F401
