"""Newton-Schulz orthogonalisation of a matrix (the polar factor used by Muon-style optimizers;
reference: ``pytorch/newton_schulz.py`` over cuSolverMp).  Quintic iteration in bf16/fp32 GEMMs."""
import torch


def newton_schulz(g: torch.Tensor, steps: int = 5, coefficients=(3.4445, -4.7750, 2.0315), eps: float = 1e-7):
    assert g.dim() == 2
    a, b, c = coefficients
    x = g.float()
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = x / (x.norm() + eps)
    for _ in range(steps):
        xxT = x @ x.t()
        x = a * x + (b * xxT + c * (xxT @ xxT)) @ x
    return (x.t() if transposed else x).to(g.dtype)
