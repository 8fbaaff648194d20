"""Operation fuser: fused plans give the same values and gradients as the unfused operations
(test model: reference ``tests/pytorch/test_fusible_ops.py``)."""
import copy

import pytest
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
    assert [getattr(p, "fusion", type(p).__name__) for p in seq2._get_plan()] == ["norm_linear", "Dropout", "linear_bias_add"]
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


def _unfused(ops, x, *extra):
    """Run copies of the operations one by one (no fusion)."""
    ref = copy.deepcopy(list(ops))
    xr = x.clone().requires_grad_()
    h, extra, outs = xr, list(extra), []
    for op in ref:
        n = getattr(op, "num_extra_inputs", 0)
        args, extra = extra[:n], extra[n:]
        h = op(h, *args)
        if getattr(op, "num_extra_outputs", 0):
            h, rest = h[0], h[1:]
            outs.extend(rest)
    return ref, xr, h, outs


def test_linear_chains_forward_and_backward_match_unfused():
    torch.manual_seed(2)
    kw = dict(dtype=torch.float32, device="cpu")
    cases = [
        ([F.BasicLinear(16, 32, **kw), F.Bias(32, **kw), F.GELU()], "linear_bias_gelu", 0),
        ([F.Linear(16, 32, **kw), F.SwiGLU(), F.AddExtraInput()], "linear_bias_swiglu_add", 1),
        ([F.BasicLinear(16, 16, **kw), F.ConstantScale(0.5), F.AddExtraInput()], "linear_scale_add", 1),
        ([F.Linear(16, 16, **kw), F.AddExtraInput()], "linear_bias_add", 1),
    ]
    for ops, name, n_extra in cases:
        for op in ops:
            for p in op.parameters():
                if p.dim() == 1:
                    torch.nn.init.normal_(p, 0.0, 0.5)   # non-zero biases
        seq = F.Sequential(*ops)
        plan = seq._get_plan()
        assert len(plan) == 1 and plan[0].fusion == name, [getattr(p, "fusion", type(p).__name__) for p in plan]
        x = torch.randn(8, 16)
        out_dim = 16 if name != "linear_bias_gelu" else 32
        extra = [torch.randn(8, 16 if "swiglu" in name or out_dim == 16 else 32).requires_grad_() for _ in range(n_extra)]
        xg = x.clone().requires_grad_()
        y = seq(xg, *extra)
        y.square().sum().backward()
        got_extra = [e.grad.clone() for e in extra]
        for e in extra:
            e.grad = None
        ref, xr, h, _ = _unfused(ops, x, *extra)
        h.square().sum().backward()
        assert torch.allclose(y, h, atol=1e-5), name
        assert torch.allclose(xg.grad, xr.grad, atol=1e-5), name
        for (n1, p1), (n2, p2) in zip(seq.named_parameters(), torch.nn.Sequential(*ref).named_parameters()):
            assert torch.allclose(p1.grad, p2.grad, atol=1e-5), (name, n1)
        for a, e in zip(got_extra, extra):
            assert torch.allclose(a, e.grad, atol=1e-6), name


def test_fork_norm_adds_branch_gradient_in_the_norm_backward():
    torch.manual_seed(3)
    kw = dict(dtype=torch.float32, device="cpu")
    ops = [F.MakeExtraOutput(), F.RMSNorm(16, **kw), F.BasicLinear(16, 16, **kw)]
    seq = F.Sequential(*ops)
    assert [getattr(p, "fusion", type(p).__name__) for p in seq._get_plan()] == ["fork_norm", "BasicLinear"]
    x = torch.randn(8, 16)
    xg = x.clone().requires_grad_()
    y, fork = seq(xg)
    (y.square().sum() + (fork * 0.3).sum()).backward()
    ref, xr, h, outs = _unfused(ops, x)
    (h.square().sum() + (outs[0] * 0.3).sum()).backward()
    assert torch.allclose(y, h, atol=1e-5) and torch.allclose(fork, x)
    assert torch.allclose(xg.grad, xr.grad, atol=1e-5)
    assert torch.allclose(seq[1].weight.grad, ref[1].weight.grad, atol=1e-5)


def test_linear_chain_under_mxfp8_autocast():
    torch.manual_seed(4)
    kw = dict(dtype=torch.float32, device="cpu")
    ops = [F.Linear(64, 128, **kw), F.GELU(), F.AddExtraInput()]
    seq = F.Sequential(*ops)
    x, r = torch.randn(32, 64), torch.randn(32, 128)
    xg = x.clone().requires_grad_()
    with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
        y = seq(xg, r)
    y.square().sum().backward()
    ref, xr, h, _ = _unfused(ops, x, r)     # high precision, unfused
    h.square().sum().backward()
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()  # noqa: E731
    assert rel(y, h) < 0.05 and rel(xg.grad, xr.grad) < 0.1 and rel(seq[0].weight.grad, ref[0].weight.grad) < 0.1
    assert rel(seq[0].bias.grad, ref[0].bias.grad) < 0.1


def test_grouped_mlp_fusion_matches_per_expert_reference():
    """GroupedLinear, ScaledSwiGLU, GroupedLinear: fused into one stand-in; forward and all gradients equal the
    per-expert loop in plain torch."""
    import transformerengine_b200 as te
    from transformerengine_b200 import fusible as F

    torch.manual_seed(0)
    G, H, FF = 3, 32, 48
    splits = [5, 0, 7]
    seq = F.Sequential(F.GroupedLinear(G, H, 2 * FF, bias=False, device="cpu", dtype=torch.float32),
                       F.ScaledSwiGLU(),
                       F.GroupedLinear(G, FF, H, bias=False, device="cpu", dtype=torch.float32))
    plan = F.fuse_operations(list(seq))
    assert len(plan) == 1 and plan[0].fusion == "grouped_mlp"
    x = torch.randn(sum(splits), H, requires_grad=True)
    probs = torch.rand(sum(splits), requires_grad=True)
    st = torch.tensor(splits)
    y = seq(x, st, probs, st)
    w = torch.randn_like(y)
    (y * w).sum().backward()
    # reference
    xr, pr = x.detach().clone().requires_grad_(), probs.detach().clone().requires_grad_()
    outs, r0 = [], 0
    w1 = [getattr(seq[0], f"weight{i}").detach().clone().requires_grad_() for i in range(G)]
    w2 = [getattr(seq[2], f"weight{i}").detach().clone().requires_grad_() for i in range(G)]
    for i, m in enumerate(splits):
        xs = xr[r0:r0 + m]
        h = xs @ w1[i].t()
        a, b = h[:, :FF], h[:, FF:]
        act = torch.nn.functional.silu(a) * b * pr[r0:r0 + m, None]
        outs.append(act @ w2[i].t())
        r0 += m
    yr = torch.cat(outs)
    torch.testing.assert_close(y, yr, rtol=1e-5, atol=1e-5)
    (yr * w).sum().backward()
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(probs.grad, pr.grad, rtol=1e-4, atol=1e-5)
    for i in (0, 2):
        torch.testing.assert_close(getattr(seq[0], f"weight{i}").grad, w1[i].grad, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(getattr(seq[2], f"weight{i}").grad, w2[i].grad, rtol=1e-4, atol=1e-5)
    # the state dict shows the experts' weights under the basic operations
    assert "0.impl.weight0" in seq.state_dict()


def test_gated_unit_variants():
    """The gated units outside the fused kernels' set against their formulas; the gate acts on the FIRST half."""
    from transformerengine_b200 import fusible as ops
    torch.manual_seed(0)
    x = (torch.randn(6, 16) * 4).requires_grad_()
    a, b = x.detach().chunk(2, dim=-1)
    torch.testing.assert_close(ops.GLU()(x), torch.sigmoid(a) * b)
    ac, bc = a.clamp(max=7.0), b.clamp(-7.0, 7.0) + 1.0
    torch.testing.assert_close(ops.ClampedSwiGLU()(x), ac * torch.sigmoid(1.702 * ac) * bc)
    torch.testing.assert_close(ops.ClampedSwiGLU(limit=2.0, alpha=1.0, glu_linear_offset=0.0)(x),
                               a.clamp(max=2.0) * torch.sigmoid(a.clamp(max=2.0)) * b.clamp(-2.0, 2.0))
    torch.testing.assert_close(ops.SiTUGLU()(x), 4 * torch.tanh(a / 4) * torch.sigmoid(a) * 25 * torch.tanh(b / 25))
    torch.testing.assert_close(ops.QGEGLU()(x), a * torch.sigmoid(1.702 * a) * b)
    torch.testing.assert_close(ops.SReGLU()(x), torch.relu(a).square() * b)
    s = torch.rand(6, requires_grad=True)
    y = ops.ScaledSReLU()(x, s)
    torch.testing.assert_close(y, torch.relu(x.detach()).square() * s.detach()[:, None])
    y.sum().backward()
    torch.testing.assert_close(s.grad, torch.relu(x.detach()).square().sum(-1))
    torch.testing.assert_close(ops.ScaledClampedQGeGLU()(x, s), ops.ClampedSwiGLU()(x) * s[:, None])
    torch.testing.assert_close(ops.ScaledSiTUGLU(beta1=2.0)(x, s), ops.SiTUGLU(beta1=2.0)(x) * s[:, None])
    # inside a Sequential: linear -> gated unit -> linear, with the scale as an extra input
    seq = ops.Sequential(ops.Linear(16, 32, bias=False, device="cpu", dtype=torch.float32),
                         ops.ScaledSiTUGLU(), ops.Linear(16, 8, bias=False, device="cpu", dtype=torch.float32))
    out = seq(x.detach(), s.detach())
    assert out.shape == (6, 8) and torch.isfinite(out).all()
    with pytest.raises(ValueError):
        ops.SiTUGLU(beta1=0.0)
    # block-interleaved layout: a1 a2 b1 b2 a3 a4 b3 b4 gives the same result as a1..a4 b1..b4, gradients included
    xi = torch.randn(6, 16, requires_grad=True)
    blocks = xi.reshape(6, 4, 2, 2)                                  # [row, pair, gate / linear, 2]
    plain = torch.cat([blocks[:, :, 0].reshape(6, 8), blocks[:, :, 1].reshape(6, 8)], -1).detach().requires_grad_()
    sc = torch.rand(6)
    for inter, ref, extra in ((ops.GLU(glu_interleave_size=2), ops.GLU(), ()),
                              (ops.SwiGLU(glu_interleave_size=2), ops.SwiGLU(), ()),
                              (ops.GEGLU(glu_interleave_size=2), ops.GEGLU(), ()),
                              (ops.ClampedSwiGLU(glu_interleave_size=2), ops.ClampedSwiGLU(), ()),
                              (ops.ScaledSwiGLU(glu_interleave_size=2), ops.ScaledSwiGLU(), (sc,)),
                              (ops.ScaledSiTUGLU(glu_interleave_size=2), ops.ScaledSiTUGLU(), (sc,))):
        xi.grad = plain.grad = None
        y, want = inter(xi, *extra), ref(plain, *extra)
        torch.testing.assert_close(y, want)
        y.square().sum().backward()
        want.square().sum().backward()
        g = plain.grad.reshape(6, 2, 4, 2).transpose(1, 2).reshape(6, 16)   # back to the interleaved layout
        torch.testing.assert_close(xi.grad, g)
    with pytest.raises(ValueError):
        ops.GLU(glu_interleave_size=3)(xi)
    with pytest.raises(ValueError):
        ops.GELU(glu_interleave_size=2)
    # an interleaved gated unit stays a basic operation (the fused linear + activation reads [gates | linear units])
    lin = ops.Linear(16, 16, bias=False, device="cpu", dtype=torch.float32)
    fused = ops.Sequential(lin, ops.SwiGLU())
    inter = ops.Sequential(lin, ops.SwiGLU(glu_interleave_size=2))
    assert any(getattr(op, "is_fused_op", False) for op in fused._get_plan())
    assert not any(getattr(op, "is_fused_op", False) for op in inter._get_plan())
    torch.testing.assert_close(inter(x.detach()), ops.SwiGLU(glu_interleave_size=2)(lin(x.detach())))


def test_user_registered_fusion_pass():
    """A fusion pass of the user's own replaces [GELU, ConstantScale] by one module; it runs before the built-in
    fusions when prepended, and the plan is rebuilt when the registry changes."""
    from transformerengine_b200 import fusible as ops
    calls = []

    class GeluTimes(torch.nn.Module):
        def __init__(self, scale):
            super().__init__()
            self.scale = scale

        def forward(self, x):
            return torch.nn.functional.gelu(x, approximate="tanh") * self.scale

    def fuse_gelu_scale(oplist, *, recipe):
        calls.append(recipe)
        out, i = [], 0
        while i < len(oplist):
            if i + 1 < len(oplist) and isinstance(oplist[i], ops.GELU) and isinstance(oplist[i + 1], ops.ConstantScale):
                out.append(GeluTimes(float(oplist[i + 1].scale)))
                i += 2
            else:
                out.append(oplist[i])
                i += 1
        return out

    seq = ops.Sequential(ops.Linear(16, 16, bias=False, device="cpu", dtype=torch.float32), ops.GELU(),
                         ops.ConstantScale(3.0))
    x = torch.randn(4, 16, requires_grad=True)
    want = seq(x)
    ops.register_forward_backward_fusion(fuse_gelu_scale, prepend=True)
    try:
        got = seq(x)
        assert calls == [None] and any(isinstance(m, GeluTimes) for m in seq._get_plan())
        torch.testing.assert_close(got, want)
        got.sum().backward()
        assert x.grad is not None
    finally:
        ops.unregister_fusion(fuse_gelu_scale)
    assert not any(isinstance(m, GeluTimes) for m in seq._get_plan())
    with pytest.raises(NotImplementedError):
        ops.register_backward_fusion(fuse_gelu_scale)
    assert ops.BasicOperation is ops.FusibleOperation


def test_backward_override_runs_the_basic_operations():
    """Under ``recipe.backward_override`` the fuser leaves the basic operations unfused (their modules run the 16-bit
    backward); the plan is rebuilt when the override changes."""
    from transformerengine_b200.common import recipe as R
    from transformerengine_b200.tensor.mxfp8 import MXFP8Quantizer
    torch.manual_seed(0)
    seq = te.ops.Sequential(te.ops.Linear(64, 64, bias=False, device="cpu", dtype=torch.float32), te.ops.GELU())
    x = torch.randn(32, 64)

    def run(recipe):
        xi = x.clone().requires_grad_()
        seq.zero_grad()
        with te.autocast(enabled=True, recipe=recipe):
            y = seq(xi)
            fused = any(getattr(op, "is_fused_op", False) for op in seq._get_plan())
        y.sum().backward()
        return y.detach(), xi.grad, seq[0].weight.grad.clone(), fused

    y0, gx0, gw0, fused0 = run(R.MXFP8BlockScaling())
    y1, gx1, gw1, fused1 = run(R.MXFP8BlockScaling(backward_override="high_precision"))
    assert fused0 and not fused1
    torch.testing.assert_close(y1, y0)
    # the 16-bit backward: gradients of the unquantized products at the forward's (quantized) pre-activation
    w = seq[0].weight.detach()
    mx = lambda t: MXFP8Quantizer()(t).dequantize()  # noqa: E731
    pre = (mx(x) @ mx(w).t()).requires_grad_()
    torch.nn.functional.gelu(pre, approximate="tanh").sum().backward()
    torch.testing.assert_close(gx1, pre.grad @ w, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gw1, pre.grad.t() @ x, rtol=1e-4, atol=1e-5)
    assert not torch.allclose(gx1, gx0, rtol=1e-4, atol=1e-5)
    assert run(R.MXFP8BlockScaling())[3]                    # fused again without the override
