"""Pass-through (identity) quantizer and tensor (the reference's module name ``pytorch/tensor/identity_tensor.py``; the classes live in ``tensor/hybrid.py``)."""
from .hybrid import *  # noqa: F401,F403
from .hybrid import IdentityQuantizer, IdentityTensor, IdentityTensorStorage  # noqa: F401
