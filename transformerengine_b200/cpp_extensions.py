"""The functional entry points that the reference exposes as ``pytorch/cpp_extensions`` (GEMM front ends), under
that module name; the implementations are in ``ops/gemm.py``."""
from __future__ import annotations

from typing import List, Optional

import torch

from .ops.gemm import as_operand, gemm_nt, general_gemm  # noqa: F401


def general_grouped_gemm(A: List, B: List, out: List[torch.Tensor], quantization_params=None, out_dtype=None, *,
                         m_splits: Optional[List[int]] = None, layout: str = "TN", bias: Optional[List] = None,
                         use_bias: bool = False, accumulate: bool = False, grad: bool = False, single_output: bool = False,
                         **_unused):
    """``out[i] = B[i] @ A[i]^T`` (layout "TN") for every group: the list form of the grouped GEMM.  With
    ``single_output`` the results are written to the row slabs (``m_splits``) of ``out[0]``."""
    assert layout in ("TN", "NN", "NT")
    if single_output:
        assert m_splits is not None
        views, r0 = [], 0
        for m in m_splits:
            views.append(out[0][r0:r0 + m])
            r0 += m
    else:
        views = out
    for i in range(len(A)):
        if views[i].numel() == 0:
            continue
        general_gemm(A[i], B[i], out_dtype=out_dtype, layout=layout, out=views[i],
                     bias=(bias[i] if (use_bias and bias is not None and not grad) else None), accumulate=accumulate,
                     grad=grad)
    return out, (None if bias is None else bias), None
