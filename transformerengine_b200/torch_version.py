"""``torch_version()`` under the reference's module name (``pytorch/torch_version.py``)."""
from .utils import torch_version  # noqa: F401
