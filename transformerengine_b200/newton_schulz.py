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

from itertools import chain, cycle, islice, repeat
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

Coeff = Tuple[float, float, float]

# Published schedules of (a, b, c) for X <- a X + (b A + c A^2) X.
_SIMPLE: List[Coeff] = [(3.4445, -4.7750, 2.0315)]                       # Muon's single triple
_QUINTIC: List[Coeff] = [(4.0848, -6.8946, 2.9270), (3.9505, -6.3029, 2.6377), (3.7418, -5.5913, 2.3037),
                         (2.8769, -3.1427, 1.2046), (2.8366, -3.0525, 1.2012)]   # tuned per step (modded-nanogpt)
# Polar Express (arXiv 2505.16932): raw minimax coefficients; Algorithm 1 divides the degree-k term by 1.01^k
_POLAR_RAW: List[Coeff] = [(8.28721201814563, -23.595886519098837, 17.300387312530933),
                           (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
                           (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
                           (3.3184196573706015, -2.488488024314874, 0.51004894012372),
                           (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
                           (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
                           (1.8750014808534479, -1.2500016453999487, 0.3750001645474248)]
_POLAR: List[Coeff] = [(a / 1.01, b / 1.01 ** 3, c / 1.01 ** 5) for a, b, c in _POLAR_RAW] + [(1.875, -1.25, 0.375)]
_SCHEDULES = {"simple": (_SIMPLE, "cycle"), "quintic": (_QUINTIC, "cycle"), "polar_express": (_POLAR, "repeat_last")}


def get_coefficient_iterator(steps: int, coefficient_sets: Sequence[Coeff], mode: str = "cycle"):
    """``steps`` triples from ``coefficient_sets``: ``"cycle"`` starts over after the last one, ``"repeat_last"``
    keeps yielding it."""
    if not coefficient_sets:
        raise ValueError("coefficient_sets must be non-empty")
    if mode == "cycle":
        it = cycle(coefficient_sets)
    elif mode == "repeat_last":
        it = chain(coefficient_sets, repeat(coefficient_sets[-1]))
    else:
        raise ValueError(f"mode must be 'cycle' or 'repeat_last', got {mode!r}")
    return islice(it, steps)


def get_coefficients(steps: int, coefficient_type: str = "quintic") -> List[Coeff]:
    """Coefficient schedule for ``steps`` iterations: ``"simple"`` (one triple, repeated), ``"quintic"`` (five tuned
    triples, cycled) or ``"polar_express"`` (eight triples, the last one repeated)."""
    if coefficient_type not in _SCHEDULES:
        raise ValueError(f"coefficient_type must be one of {sorted(_SCHEDULES)}, got {coefficient_type!r}")
    sets, mode = _SCHEDULES[coefficient_type]
    return list(get_coefficient_iterator(steps, sets, mode))


class CusolverMpCtx:
    """Context of the distributed iteration (the name is the reference's, where it wraps a cuSolverMp grid; here
    the products run on this library's GEMM and the only communication is the all-reduce of the small Gram matrix,
    so the context just pins the process group).  ``newton_schulz(x, ctx, num_iterations, coefficients)`` then
    orthogonalises IN PLACE a matrix whose COLUMNS are spread over the group's ranks."""

    def __init__(self, group) -> None:
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialized before creating CusolverMpCtx")
        self.group = group
        self.nranks, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.rank < 0:
            raise RuntimeError("this process is not a member of the group")

    def destroy(self) -> None:
        self.group = None


def _mm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M, K] @ b[N, K]^T in fp32 out; bf16 operands on CUDA use the library GEMM."""
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16) and a.dtype == b.dtype and a.shape[1] % 8 == 0:
        from . import ops

        return ops.gemm_nt(a.contiguous(), b.contiguous(), out_dtype=torch.float32)
    return a.float() @ b.float().t()


def newton_schulz(g: torch.Tensor, steps=5, coefficients=(3.4445, -4.7750, 2.0315),
                  eps: float = 1e-7, group=None, partition_dim: Optional[int] = None,
                  compute_dtype: torch.dtype = torch.bfloat16, num_iterations: Optional[int] = None,
                  ctx: Optional[CusolverMpCtx] = None):
    """Approximate polar factor of ``g`` (2-D).  ``group`` / ``partition_dim``: ``g`` is this rank's shard of a
    matrix split along ``partition_dim`` (which must be the long dimension of the full matrix).
    ``coefficients``: one ``(a, b, c)`` triple for every step, or a sequence of triples, one per step
    (``get_coefficients``).  Returns the result.

    Reference call form ``newton_schulz(x, ctx, num_iterations=5, coefficients=None)`` with a ``CusolverMpCtx``:
    the columns of ``x`` are spread over the context's group, the default schedule is ``get_coefficients(n)``,
    ``x`` is overwritten and nothing is returned."""
    assert g.dim() == 2
    if isinstance(steps, CusolverMpCtx):
        # positional reference form (x, ctx, num_iterations, coefficients): shift the arguments into place
        ctx = steps
        ref_n, ref_coeffs = coefficients, eps
        steps = ref_n if isinstance(ref_n, int) else 5
        coefficients = ref_coeffs if isinstance(ref_coeffs, (list, tuple)) else (
            None if isinstance(ref_n, int) or tuple(ref_n) == _SIMPLE[0] else ref_n)
        eps = 1e-7
    if ctx is not None:
        if num_iterations is not None:
            steps = num_iterations
        if coefficients is None or (len(coefficients) == 3 and not isinstance(coefficients[0], (tuple, list))
                                    and tuple(coefficients) == _SIMPLE[0]):
            coefficients = get_coefficients(steps)       # the reference's default schedule
        if g.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"expected a float32 or bfloat16 tensor, got {g.dtype}")
        if ctx.group is None:
            raise RuntimeError("the context was destroyed")
        out = newton_schulz(g, steps, coefficients, eps, ctx.group if ctx.nranks > 1 else None,
                            1 if ctx.nranks > 1 else None, compute_dtype)
        g.copy_(out)
        return None
    if num_iterations is not None:
        steps = num_iterations
    if len(coefficients) == 3 and not isinstance(coefficients[0], (tuple, list)):
        schedule = [tuple(coefficients)] * steps
    else:
        schedule = [tuple(t) for t in coefficients]
        if len(schedule) != steps or any(len(t) != 3 for t in schedule):
            raise ValueError(f"expected {steps} coefficient triples, got {len(schedule)}")
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
    for a, b, c in schedule:
        xc = x.to(cd)
        gram = _mm_nt(xc, xc)                      # [short, short] partial Gram matrix
        if world > 1:
            dist.all_reduce(gram, group=group)
        gc = gram.to(cd)
        poly = b * gram + c * _mm_nt(gc, gc)       # gram is symmetric: G G^T = G^2
        x = a * x + _mm_nt(poly.to(cd), xc.t().contiguous())
    out = x.t() if long_dim == 0 else x
    return out.to(g.dtype)
