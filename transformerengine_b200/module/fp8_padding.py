"""``Fp8Padding`` under the reference's module name (``pytorch/module/fp8_padding.py``)."""
from ..modules.grouped_linear import *  # noqa: F401,F403
from ..modules.grouped_linear import Fp8Padding  # noqa: F401
