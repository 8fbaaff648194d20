"""Grouped tensors (the reference's module name ``pytorch/tensor/grouped_tensor.py``; the classes live in ``tensor/grouped.py``)."""
from .grouped import *  # noqa: F401,F403
from .grouped import GroupedTensor, GroupedTensorStorage  # noqa: F401
