"""Newton-Schulz orthogonalisation of a matrix (the polar factor used by Muon-style optimizers;
reference: ``pytorch/newton_schulz.py`` over cuSolverMp, a DISTRIBUTED iteration on a sharded matrix).

Quintic iteration ``X <- a X + (b A + c A^2) X`` with ``A = X X^T``.  With ``group`` the matrix is sharded
along its LONG dimension (``partition_dim``): every rank holds a slice ``X_r`` and

    A = sum_r X_r X_r^T          one all-reduce of the small Gram matrix per step,
    X_r <- a X_r + (b A + c A^2) X_r      local,

so each step moves ``min(m, n)^2`` numbers per rank however large the matrix is.  On CUDA the products
run on this library's tcgen05 GEMM in bf16 with fp32 accumulation (Gram matrices are kept in fp32).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist


def _mm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M, K] @ b[N, K]^T in fp32 out; bf16 operands on CUDA use the library GEMM."""
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16) and a.dtype == b.dtype and a.shape[1] % 8 == 0:
        from . import ops

        return ops.gemm_nt(a.contiguous(), b.contiguous(), out_dtype=torch.float32)
    return a.float() @ b.float().t()


def newton_schulz(g: torch.Tensor, steps: int = 5, coefficients: Sequence[float] = (3.4445, -4.7750, 2.0315),
                  eps: float = 1e-7, group=None, partition_dim: Optional[int] = None,
                  compute_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Approximate polar factor of ``g`` (2-D).  ``group`` / ``partition_dim``: ``g`` is this rank's shard of a
    matrix split along ``partition_dim`` (which must be the long dimension of the full matrix)."""
    assert g.dim() == 2
    a, b, c = coefficients
    world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    if world > 1:
        assert partition_dim in (0, 1), "a sharded matrix needs partition_dim"
        long_dim = partition_dim
    else:
        long_dim = 1 if g.shape[1] >= g.shape[0] else 0
    # work on X [short, long_local]: rows = the short dimension
    x = (g.t() if long_dim == 0 else g).float()
    if world > 1:
        assert x.shape[0] <= x.shape[1] * world, "partition_dim must be the long dimension of the full matrix"
    sq = x.square().sum()
    if world > 1:
        dist.all_reduce(sq, group=group)
    x = x / (sq.sqrt() + eps)
    cd = compute_dtype if x.is_cuda else torch.float32
    for _ in range(steps):
        xc = x.to(cd)
        gram = _mm_nt(xc, xc)                      # [short, short] partial Gram matrix
        if world > 1:
            dist.all_reduce(gram, group=group)
        gc = gram.to(cd)
        poly = b * gram + c * _mm_nt(gc, gc)       # gram is symmetric: G G^T = G^2
        x = a * x + _mm_nt(poly.to(cd), xc.t().contiguous())
    out = x.t() if long_dim == 0 else x
    return out.to(g.dtype)
