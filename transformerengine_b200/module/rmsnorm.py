"""``RMSNorm`` under the reference's module name (``pytorch/module/rmsnorm.py``)."""
from ..modules.layernorm_linear import *  # noqa: F401,F403
from ..modules.layernorm_linear import RMSNorm  # noqa: F401
