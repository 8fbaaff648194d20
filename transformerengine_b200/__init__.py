"""B200-native low-precision transformer library (PyTorch front end)."""
from .common import recipe  # noqa: F401
from . import ops  # noqa: F401
from .ops import check_status  # noqa: F401
from . import tensor  # noqa: F401
