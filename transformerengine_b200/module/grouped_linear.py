"""``GroupedLinear`` under the reference's module name (``pytorch/module/grouped_linear.py``)."""
from ..modules.grouped_linear import *  # noqa: F401,F403
from ..modules.grouped_linear import GroupedLinear  # noqa: F401
