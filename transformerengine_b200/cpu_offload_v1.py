"""The reference keeps two generations of its activation offload (``pytorch/cpu_offload_v1.py`` is selected with
``NVTE_CPU_OFFLOAD_V1=1``); here there is one implementation, and this module name resolves to it."""
from .cpu_offload import *  # noqa: F401,F403
from .cpu_offload import (get_cpu_offload_context, is_cpu_offload_enabled, mark_activation_offload,  # noqa: F401
                          mark_not_offload)
