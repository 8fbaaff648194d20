"""``Fp8Unpadding`` under the reference's module name (``pytorch/module/fp8_unpadding.py``)."""
from ..modules.grouped_linear import *  # noqa: F401,F403
from ..modules.grouped_linear import Fp8Unpadding  # noqa: F401
