"""``TransformerEngineBaseModule, get_default_init_method, initialize_ub, destroy_ub, is_ub_initialized`` under the reference's module name (``pytorch/module/base.py``)."""
from ..modules.base import *  # noqa: F401,F403
from ..modules.base import TransformerEngineBaseModule, get_default_init_method, initialize_ub, destroy_ub, is_ub_initialized  # noqa: F401
