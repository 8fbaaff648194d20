"""``Float8TensorStorage`` under the reference's module name."""
from . import Float8TensorStorage  # noqa: F401
