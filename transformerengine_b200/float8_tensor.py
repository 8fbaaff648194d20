"""Legacy module name (reference: ``pytorch/float8_tensor.py``)."""
from .tensor.float8 import Float8Tensor  # noqa: F401
