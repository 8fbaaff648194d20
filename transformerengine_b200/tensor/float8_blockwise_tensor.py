"""Block-scaled FP8 tensors and quantizer (the reference's module name ``pytorch/tensor/float8_blockwise_tensor.py``; the classes live in ``tensor/blockwise.py``)."""
from .blockwise import *  # noqa: F401,F403
from .blockwise import Float8BlockQuantizer, Float8BlockwiseQTensor, Float8BlockwiseQTensorStorage  # noqa: F401
