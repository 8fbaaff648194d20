"""``MXFP8TensorStorage`` under the reference's module name."""
from . import MXFP8TensorStorage  # noqa: F401
