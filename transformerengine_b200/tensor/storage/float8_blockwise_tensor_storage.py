"""``Float8BlockwiseQTensorStorage`` under the reference's module name."""
from . import Float8BlockwiseQTensorStorage  # noqa: F401
