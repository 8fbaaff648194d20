"""MoE router functions under the reference's module name (``pytorch/router.py``)."""
from .moe.router import (QBHistogramMode, RoutingMapFormat, fused_compute_score_for_moe_aux_loss,  # noqa: F401
                         fused_moe_aux_loss, fused_topk_with_score_function)
