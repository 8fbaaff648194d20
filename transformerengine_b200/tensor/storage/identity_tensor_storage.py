"""``IdentityTensorStorage`` under the reference's module name."""
from . import IdentityTensorStorage  # noqa: F401
