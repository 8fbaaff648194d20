"""``HybridQuantizedTensorStorage`` under the reference's module name."""
from . import HybridQuantizedTensorStorage  # noqa: F401
