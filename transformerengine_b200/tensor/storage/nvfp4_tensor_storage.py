"""``NVFP4TensorStorage`` under the reference's module name."""
from . import NVFP4TensorStorage  # noqa: F401
