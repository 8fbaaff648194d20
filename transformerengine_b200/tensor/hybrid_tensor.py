"""Per-direction (hybrid) quantized tensors (the reference's module name ``pytorch/tensor/hybrid_tensor.py``; the classes live in ``tensor/hybrid.py``)."""
from .hybrid import *  # noqa: F401,F403
from .hybrid import HybridQuantizedTensor, HybridQuantizedTensorStorage, HybridQuantizer  # noqa: F401
