"""The ``torch.library`` operators: eager results and gradients against plain PyTorch, and a block traced by
``torch.compile`` as ONE graph (``fullgraph=True``: any graph break fails the test)."""
import pytest
import torch

import transformerengine_b200.compile_ops as cops


def _ref_block(x, g, w1, w2, freqs):
    xf = x.float()
    h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()).to(x.dtype)
    u = h @ w1.t()
    n = u.shape[-1] // 2
    a = torch.nn.functional.silu(u[..., :n]) * u[..., n:]
    return a @ w2.t()


def _block(x, g, w1, w2, freqs):
    h = cops.rmsnorm(x, g, 1e-5)
    return cops.linear(cops.swiglu(cops.linear(h, w1)), w2)


def _inputs():
    torch.manual_seed(0)
    x = torch.randn(6, 4, 32, requires_grad=True)
    g = (torch.rand(32) + 0.5).requires_grad_()
    w1 = (torch.randn(48, 32) * 0.1).requires_grad_()
    w2 = (torch.randn(32, 24) * 0.1).requires_grad_()
    return x, g, w1, w2, None


def test_operators_match_pytorch_in_eager_mode():
    args = _inputs()
    y = _block(*args)
    yr = _ref_block(*[a.detach().clone().requires_grad_() if a is not None else None for a in args])
    torch.testing.assert_close(y, yr, rtol=1e-4, atol=1e-5)
    w = torch.randn_like(y)
    grads = torch.autograd.grad((y * w).sum(), args[:4])
    ref_args = [a.detach().clone().requires_grad_() for a in args[:4]]
    gr = torch.autograd.grad((_ref_block(*ref_args, None) * w).sum(), ref_args)
    for a, b in zip(grads, gr):
        torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-4)


def test_layernorm_rope_and_cross_entropy_operators():
    torch.manual_seed(1)
    x = torch.randn(5, 16, requires_grad=True)
    g, b = torch.rand(16, requires_grad=True), torch.randn(16, requires_grad=True)
    y = cops.layernorm(x, g, b, 1e-5)
    yr = torch.nn.functional.layer_norm(x, (16,), g, b, 1e-5)
    torch.testing.assert_close(y, yr, rtol=1e-4, atol=1e-5)
    gx = torch.autograd.grad(y.square().sum(), (x, g, b))
    gr = torch.autograd.grad(yr.square().sum(), (x, g, b))
    for a_, b_ in zip(gx, gr):
        torch.testing.assert_close(a_, b_, rtol=1e-3, atol=1e-4)
    # rope: rotating and rotating back with the transposed map is the identity on the gradient path
    from transformerengine_b200 import ops

    q = torch.randn(7, 2, 3, 16, requires_grad=True)
    f = ops.rope_freqs(torch.arange(7), 16, 10000.0, False)
    r = cops.rope(q, f)
    assert r.shape == q.shape
    (gq,) = torch.autograd.grad(r.sum(), q)
    assert torch.isfinite(gq).all()
    torch.testing.assert_close(r.norm(), q.norm(), rtol=1e-4, atol=1e-4)      # a rotation keeps the norm
    logits = torch.randn(4, 3, 11, requires_grad=True)
    tgt = torch.randint(0, 11, (4, 3))
    tgt[1, 1] = -100
    loss = cops.cross_entropy(logits, tgt)
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 11), tgt.reshape(-1), reduction="none").reshape(4, 3)
    torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-5)
    (gl,) = torch.autograd.grad(loss.sum(), logits)
    (glr,) = torch.autograd.grad(ref.sum(), logits)
    torch.testing.assert_close(gl, glr, rtol=1e-4, atol=1e-5)


def test_block_compiles_as_one_graph():
    args = _inputs()
    compiled = torch.compile(_block, backend="aot_eager", fullgraph=True)
    y = compiled(*args)
    torch.testing.assert_close(y, _block(*args), rtol=1e-5, atol=1e-6)
    (y.sum()).backward()
    assert args[0].grad is not None and args[2].grad is not None
    # the traced graph holds the library's operators as single nodes
    from torch._dynamo.testing import EagerAndRecordGraphs

    rec = EagerAndRecordGraphs()
    torch.compile(_block, backend=rec, fullgraph=True)(*[a.detach() if a is not None else None for a in args])
    text = rec.graphs[0].print_readable(print_output=False)
    assert "teb200.norm_fwd" in text and "teb200.gemm_nt" in text and "teb200.activation_fwd" in text
