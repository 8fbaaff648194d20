"""``Linear`` under the reference's module name (``pytorch/module/linear.py``)."""
from ..modules.linear import *  # noqa: F401,F403
from ..modules.linear import Linear  # noqa: F401
