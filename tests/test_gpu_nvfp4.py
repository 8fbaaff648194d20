"""NVFP4 CUDA kernels against the pure-PyTorch oracle (test model: reference
``tests/pytorch/nvfp4/test_nvfp4_quantize_exact.py``, ``test_nvfp4_rht_quantize_exact.py``,
``test_nvfp4_sr_quantize.py``, ``test_nvfp4_gemm_exact.py``)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle(x, **kw):
    from transformerengine_b200.ops import quantize as qz

    return qz.quantize_nvfp4(x.cpu(), **kw)


@pytest.mark.parametrize("shape", [(128, 256), (256, 512), (48, 96)])
@pytest.mark.parametrize("with_rht", [False, True])
@pytest.mark.parametrize("with_2d", [False, True])
def test_quantize_matches_oracle(shape, with_rht, with_2d):
    from transformerengine_b200.ops import quantize as qz

    if with_rht and with_2d:
        pytest.skip("the recipe never combines 2-D weight blocks with the Hadamard transform")
    torch.manual_seed(0)
    x = (torch.randn(*shape, device="cuda") * 3).to(torch.bfloat16)
    got = qz.quantize_nvfp4(x, with_rht=with_rht, with_2d=with_2d)
    ref = _oracle(x, with_rht=with_rht, with_2d=with_2d)
    names = ["row_data", "row_scale", "amax_row", "col_data", "col_scale", "amax_col"]
    for n, g, r in zip(names, got, ref):
        g, r = g.cpu(), r.cpu()
        if "amax" in n:
            assert torch.allclose(g.float(), r.float(), rtol=1e-6), n
        else:
            mism = (g.reshape(-1) != r.reshape(-1)).float().mean().item()
            # the Hadamard butterflies add in a different order than the oracle's matmul: a few
            # values on a rounding boundary may move by one code
            assert mism <= (2e-3 if with_rht and n.startswith("col") else 0.0), (n, mism)


def test_dequantize_roundtrip_and_stochastic_rounding_is_unbiased():
    from transformerengine_b200.ops import quantize as qz

    torch.manual_seed(1)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    rd, rs, ar, _, _, _ = qz.quantize_nvfp4(x, columnwise=False)
    dq = qz.dequantize_nvfp4(rd, rs, ar, 256, 512, torch.float32)
    rel = (dq - x.float()).norm() / x.float().norm()
    assert rel < 0.12
    acc = torch.zeros_like(dq)
    n = 64
    for _ in range(n):
        d, s, a, _, _, _ = qz.quantize_nvfp4(x, columnwise=False, stochastic_rounding=True)
        acc += qz.dequantize_nvfp4(d, s, a, 256, 512, torch.float32)
    mean_err = (acc / n - x.float()).norm() / x.float().norm()
    assert mean_err < rel * 0.35, (mean_err.item(), rel.item())


def test_nvfp4_gemm_matches_dequantized_matmul():
    import transformerengine_b200 as te
    from transformerengine_b200 import ops
    from transformerengine_b200.tensor.nvfp4 import NVFP4Quantizer

    torch.manual_seed(2)
    M, N, K = 256, 384, 512
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    q = NVFP4Quantizer(columnwise=False)
    qa, qb = q(a), q(b)
    out = ops.gemm_nt(ops.as_operand(qa), ops.as_operand(qb), out_dtype=torch.float32)
    te.ops.check_status()
    ref = qa.dequantize().float() @ qb.dequantize().float().t()
    err = (out - ref).abs().max().item() / ref.abs().max().item()
    assert err < 5e-3, err


def test_linear_under_nvfp4_recipe():
    import transformerengine_b200 as te

    torch.manual_seed(3)
    lin = te.Linear(512, 512, bias=False, params_dtype=torch.bfloat16, device="cuda")
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    with te.autocast(enabled=True, recipe=te.recipe.NVFP4BlockScaling()):
        y = lin(x)
    y.float().square().mean().backward()
    te.ops.check_status()
    ref = x.detach().float() @ lin.weight.detach().float().t()
    rel = (y.float() - ref).norm() / ref.norm()
    assert rel < 0.2, rel.item()
    assert torch.isfinite(x.grad.float()).all() and torch.isfinite(lin.weight.grad.float()).all()


@pytest.mark.parametrize("shape", [(8192, 4096), (1040, 272)])
@pytest.mark.parametrize("with_rht", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_one_pass_row_and_column_kernel_is_bitwise_the_two_single_copy_kernels(shape, with_rht, dtype):
    """Asking for both copies runs the kernel that reads the input once; asking for one copy at a time runs the
    single-copy kernels.  Same functions on the same values: every byte must agree (partial tiles included)."""
    from transformerengine_b200.ops import quantize as qz

    torch.manual_seed(1)
    x = (torch.randn(*shape, device="cuda") * 2).to(dtype)
    both = qz.quantize_nvfp4(x, with_rht=with_rht)
    row = qz.quantize_nvfp4(x, rowwise=True, columnwise=False, with_rht=with_rht)
    col = qz.quantize_nvfp4(x, rowwise=False, columnwise=True, with_rht=with_rht)
    assert torch.equal(both[0], row[0]) and torch.equal(both[1], row[1]) and torch.equal(both[2], row[2])
    assert torch.equal(both[3], col[3]) and torch.equal(both[4], col[4]) and torch.equal(both[5], col[5])
