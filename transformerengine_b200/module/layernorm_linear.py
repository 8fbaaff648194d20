"""``LayerNormLinear`` under the reference's module name (``pytorch/module/layernorm_linear.py``)."""
from ..modules.layernorm_linear import *  # noqa: F401,F403
from ..modules.layernorm_linear import LayerNormLinear  # noqa: F401
