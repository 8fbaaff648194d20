"""MoE token permutation under the reference's module name (``pytorch/permutation.py``)."""
from .moe.permutation import *  # noqa: F401,F403
from .moe.permutation import (moe_permute, moe_permute_and_pad_with_probs, moe_permute_with_probs,  # noqa: F401
                              moe_sort_chunks_by_index, moe_sort_chunks_by_index_with_probs, moe_unpermute)
