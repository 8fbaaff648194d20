"""``LayerNorm`` under the reference's module name (``pytorch/module/layernorm.py``)."""
from ..modules.layernorm_linear import *  # noqa: F401,F403
from ..modules.layernorm_linear import LayerNorm  # noqa: F401
