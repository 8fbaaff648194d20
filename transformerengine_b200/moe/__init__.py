"""Mixture-of-experts building blocks: router, token permutation, grouped linear, expert parallel."""
from .router import (fused_topk_with_score_function, fused_compute_score_for_moe_aux_loss, fused_moe_aux_loss,
                     RoutingMapFormat, QBHistogramMode)
from .permutation import (moe_permute, moe_permute_with_probs, moe_permute_and_pad_with_probs, moe_unpermute,
                          moe_sort_chunks_by_index, moe_sort_chunks_by_index_with_probs)
