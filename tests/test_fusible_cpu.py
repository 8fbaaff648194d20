"""Operation fuser: fused plans give the same values and gradients as the unfused operations
(test model: reference ``tests/pytorch/test_fusible_ops.py``)."""
import copy

import torch

import transformerengine_b200 as te
from transformerengine_b200 import fusible as F
from transformerengine_b200.fusible.sequential import fuse_operations


def _run(seq, x, *extra):
    x = x.clone().requires_grad_()
    y = seq(x, *extra)
    y0 = y[0] if isinstance(y, tuple) else y
    y0.square().sum().backward()
    return y, x.grad, {n: p.grad.clone() for n, p in seq.named_parameters()}


def test_norm_mlp_fusion_matches_unfused():
    torch.manual_seed(0)
    ops = [F.RMSNorm(32, dtype=torch.float32, device="cpu"),
           F.BasicLinear(32, 128, dtype=torch.float32, device="cpu"), F.SwiGLU(),
           F.BasicLinear(64, 32, dtype=torch.float32, device="cpu")]
    seq = F.Sequential(*ops)
    plan = seq._get_plan()
    assert len(plan) == 1 and plan[0].fusion == "norm_mlp"
    x = torch.randn(6, 32)
    y, dx, grads = _run(seq, x)
    # unfused: call the operations one by one
    ref_ops = copy.deepcopy(ops)
    xr = x.clone().requires_grad_()
    h = xr
    for op in ref_ops:
        h = op(h)
    h.square().sum().backward()
    assert torch.allclose(y, h, atol=1e-5)
    assert torch.allclose(dx, xr.grad, atol=1e-5)
    assert torch.allclose(grads["1.weight"], ref_ops[1].weight.grad, atol=1e-5)
    assert torch.allclose(grads["0.weight"], ref_ops[0].weight.grad, atol=1e-5)
    assert set(dict(seq.named_parameters())) == {"0.weight", "1.weight", "3.weight"}


def test_norm_linear_and_residual_fusion():
    torch.manual_seed(1)
    seq = F.Sequential(F.LayerNorm(16, dtype=torch.float32, device="cpu"),
                       F.Linear(16, 16, dtype=torch.float32, device="cpu"), F.GELU(),
                       F.Linear(16, 16, dtype=torch.float32, device="cpu"), F.AddExtraInput(), F.MakeExtraOutput())
    kinds = [getattr(p, "fusion", type(p).__name__) for p in seq._get_plan()]
    assert kinds == ["norm_mlp", "AddExtraInput", "MakeExtraOutput"]
    seq2 = F.Sequential(seq[0], seq[1], F.Dropout(0.0), seq[3], F.AddExtraInput())
    assert [getattr(p, "fusion", type(p).__name__) for p in seq2._get_plan()] == ["norm_linear", "Dropout", "linear_add"]
    xx, rr = torch.randn(4, 16), torch.randn(4, 16)
    assert torch.allclose(seq2(xx, rr), seq[3](seq[1](seq[0](xx))) + rr, atol=1e-5)
    x, res = torch.randn(4, 16), torch.randn(4, 16)
    (y, y2), dx, _ = _run(seq, x, res)
    ln, l1, act, l2 = seq[0], seq[1], seq[2], seq[3]
    ref = l2(act(l1(ln(x)))) + res
    assert torch.allclose(y, ref, atol=1e-5) and y2 is y


def test_quantize_op_under_autocast():
    x = torch.randn(8, 64)
    q = F.Quantize()
    assert q(x) is x
    with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
        y = q(x)
    assert y.shape == x.shape and not torch.equal(y, x) and (y - x).abs().max() < 0.3
