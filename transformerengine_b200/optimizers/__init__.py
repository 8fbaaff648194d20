"""Fused optimizers under the reference's package name (``pytorch/optimizers``); the implementations live in
``optim/``."""
from ..optim import *  # noqa: F401,F403
from ..optim import FusedAdam, FusedSGD  # noqa: F401
try:
    from ..optim import multi_tensor_applier  # noqa: F401
except ImportError:  # pragma: no cover
    pass
