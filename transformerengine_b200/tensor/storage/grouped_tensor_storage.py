"""``GroupedTensorStorage`` under the reference's module name."""
from . import GroupedTensorStorage  # noqa: F401
