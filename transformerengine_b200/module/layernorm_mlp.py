"""``LayerNormMLP`` under the reference's module name (``pytorch/module/layernorm_mlp.py``)."""
from ..modules.layernorm_mlp import *  # noqa: F401,F403
from ..modules.layernorm_mlp import LayerNormMLP  # noqa: F401
