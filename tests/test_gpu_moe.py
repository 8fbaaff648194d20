"""MoE CUDA kernels (router, permutation), grouped GEMM and the Mixtral block on the GPU against
the pure-PyTorch path (test model: reference ``tests/pytorch/test_fused_router.py``,
``test_permutation.py``, ``test_grouped_linear.py``)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("score_function", ["softmax", "sigmoid", "sqrtsoftplus"])
@pytest.mark.parametrize("pre", [False, True])
@pytest.mark.parametrize("E,topk", [(8, 2), (64, 6), (256, 8)])
def test_router_kernel_matches_torch(score_function, pre, E, topk):
    import transformerengine_b200 as te

    if pre and score_function != "softmax":
        pytest.skip("pre-softmax only applies to the softmax score function")
    torch.manual_seed(0)
    T = 333
    logits = torch.randn(T, E, device="cuda") * 2
    bias = torch.randn(E, device="cuda") * 0.1 if score_function != "softmax" else None
    lg = logits.clone().requires_grad_()
    probs, rmap = te.fused_topk_with_score_function(lg, topk, pre, None, None, 1.5, score_function, bias)
    lc = logits.cpu().clone().requires_grad_()
    rp, rm = te.fused_topk_with_score_function(lc, topk, pre, None, None, 1.5, score_function,
                                               None if bias is None else bias.cpu())
    assert torch.equal(rmap.cpu(), rm)
    assert torch.allclose(probs.cpu(), rp, atol=2e-5, rtol=1e-4)
    g = torch.randn(T, E)
    (probs * g.cuda()).sum().backward()
    (rp * g).sum().backward()
    assert torch.allclose(lg.grad.cpu(), lc.grad, atol=5e-5, rtol=1e-3)


def test_permute_unpermute_kernels():
    import transformerengine_b200 as te

    torch.manual_seed(1)
    T, E, H, k = 257, 8, 256, 2
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    probs, rmap = te.fused_topk_with_score_function(logits, k)
    xg = x.clone().requires_grad_()
    pg = probs.clone().requires_grad_()
    out, pp, dest, _, padded = te.moe_permute_and_pad_with_probs(xg, pg, rmap, rmap.sum(0), 32)
    y = te.moe_unpermute(out * 2, dest, pg)
    y.float().sum().backward()
    # CPU reference through the index_put path
    xc = x.cpu().float().requires_grad_()
    pc = probs.cpu().clone().requires_grad_()
    outc, ppc, destc, _, paddedc = te.moe_permute_and_pad_with_probs(xc, pc, rmap.cpu(), rmap.cpu().sum(0), 32)
    yc = te.moe_unpermute(outc * 2, destc, pc)
    yc.sum().backward()
    assert torch.equal(dest.cpu(), destc) and torch.equal(padded.cpu(), paddedc)
    assert torch.allclose(out.cpu().float(), outc, atol=1e-6)
    assert torch.allclose(pp.cpu(), ppc, atol=1e-6)
    assert torch.allclose(y.cpu().float(), yc, atol=0.06, rtol=0.02)
    assert torch.allclose(xg.grad.cpu().float(), xc.grad, atol=0.03, rtol=0.02)
    assert torch.allclose(pg.grad.cpu(), pc.grad, atol=0.5, rtol=0.02)


def test_grouped_linear_mxfp8_matches_loop():
    import transformerengine_b200 as te

    torch.manual_seed(2)
    G, K, N = 4, 256, 384
    m_splits = [128, 256, 0, 128]
    gl = te.GroupedLinear(G, K, N, bias=False, params_dtype=torch.bfloat16, device="cuda")
    x = torch.randn(sum(m_splits), K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
        y = gl(x, m_splits)
    y.float().square().mean().backward()
    te.ops.check_status()
    ref, pos = [], 0
    for g, m in enumerate(m_splits):
        w = getattr(gl, f"weight{g}")
        ref.append(x[pos:pos + m].detach().float() @ w.detach().float().t())
        pos += m
    ref = torch.cat(ref)
    rel = (y.float() - ref).norm() / ref.norm()
    assert rel < 0.06, rel.item()
    assert torch.isfinite(x.grad.float()).all()
    # gradients (one quantization of grad_output, grouped dgrad, slab-view wgrads) against an fp32 loop
    xr = x.detach().float().requires_grad_()
    ws = [getattr(gl, f"weight{g}").detach().float().requires_grad_() for g in range(G)]
    outs, pos = [], 0
    for g, m in enumerate(m_splits):
        outs.append(xr[pos:pos + m] @ ws[g].t())
        pos += m
    torch.cat(outs).square().mean().backward()
    rel_dx = (x.grad.float() - xr.grad).norm() / xr.grad.norm()
    assert rel_dx < 0.08, rel_dx.item()
    for g, m in enumerate(m_splits):
        gw = getattr(gl, f"weight{g}").grad.float()
        if m == 0:
            assert gw.abs().max() == 0
        else:
            rel_dw = (gw - ws[g].grad).norm() / ws[g].grad.norm()
            assert rel_dw < 0.08, (g, rel_dw.item())
    # a second step reuses the cached stacked operands; an optimizer step invalidates them
    gl.zero_grad(set_to_none=True)
    with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
        y2 = gl(x.detach(), m_splits)
    assert torch.equal(y2, y.detach())


def test_mixtral_tiny_trains_on_gpu():
    import transformerengine_b200 as te
    from transformerengine_b200.models.mixtral import MixtralConfig, MixtralModel

    torch.manual_seed(3)
    cfg = MixtralConfig.tiny(hidden_size=256, num_heads=2, num_kv_heads=1, ffn_hidden_size=256, pad_align=128)
    model = MixtralModel(cfg, device="cuda")
    tokens = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    with te.autocast(enabled=True, recipe=te.recipe.MXFP8BlockScaling()):
        loss = model(tokens, tokens)
    loss.backward()
    te.ops.check_status()
    assert torch.isfinite(loss) and loss.item() > 0
    gn = sum(p.grad.float().norm() ** 2 for p in model.parameters() if p.grad is not None)
    assert torch.isfinite(gn) and gn > 0
