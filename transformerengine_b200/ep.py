"""Expert-parallel dispatch / combine under the reference's module name (``pytorch/ep.py``)."""
from .parallel.expert_parallel import *  # noqa: F401,F403
from .parallel.expert_parallel import ep_combine, ep_dispatch  # noqa: F401
