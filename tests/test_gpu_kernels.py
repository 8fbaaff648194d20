"""CUDA kernels against the pure-PyTorch fp32 reference of the same op."""
import pytest
import torch

import transformerengine_b200 as te
from transformerengine_b200 import ops
from transformerengine_b200.ops import quantize as qz
from transformerengine_b200.ops.ref import quant as Q
from transformerengine_b200.tensor import MXFP8Quantizer, Float8Quantizer, Float8CurrentScalingQuantizer

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_linear_fp32_parameters_keep_fp32_math():
    """fp32 parameters and activations are not rounded to bf16 on the way into the GEMM."""
    torch.manual_seed(0)
    lin = te.Linear(384, 640, params_dtype=torch.float32, device=DEV)
    x = torch.randn(200, 384, device=DEV, requires_grad=True)
    y = lin(x)
    y.square().sum().backward()
    xr = x.detach().clone().requires_grad_()
    w, b = lin.weight.detach().clone().requires_grad_(), lin.bias.detach().clone().requires_grad_()
    yr = torch.nn.functional.linear(xr.double(), w.double(), b.double())
    yr.square().sum().backward()
    assert _rel(y, yr) < 1e-5
    assert _rel(x.grad, xr.grad) < 1e-5 and _rel(lin.weight.grad, w.grad) < 1e-5


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 520, 264), (1024, 1024, 4096), (64, 96, 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_16bit(M, N, K, dtype):
    a = torch.randn(M, K, device=DEV, dtype=dtype)
    b = torch.randn(N, K, device=DEV, dtype=dtype)
    ref = a.float() @ b.float().t()
    out = ops.gemm_nt(a, b, out_dtype=dtype)
    te.check_status()
    assert _rel(out, ref) < 1e-2
    out32 = ops.gemm_nt(a, b, out_dtype=torch.float32)
    assert _rel(out32, ref) < 1e-5 * K ** 0.5 + 1e-4


def test_gemm_16bit_bias_accumulate():
    M, N, K = 384, 640, 512
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t() + bias.float()
    out = ops.gemm_nt(a, b, out_dtype=torch.float32, bias=bias)
    assert _rel(out, ref) < 1e-3
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref2 = acc + a.float() @ b.float().t()
    ops.gemm_nt(a, b, out=acc, accumulate=True)
    te.check_status()
    assert _rel(acc, ref2) < 1e-3


def test_gemm_16bit_gelu_epilogues():
    M, N, K = 256, 256, 128
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16) * 0.2
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.2
    pre = a.float() @ b.float().t()
    aux = torch.empty(M, N, device=DEV, dtype=torch.float32)
    out = ops.gemm_nt(a, b, out_dtype=torch.float32, epilogue=ops.gemm.EPI_GELU, aux=aux)
    assert _rel(aux, pre) < 1e-3
    assert _rel(out, torch.nn.functional.gelu(pre, approximate="tanh")) < 1e-3


def test_gemm_mn_major_operands():
    M, N, K = 256, 384, 320
    at = torch.randn(K, M, device=DEV, dtype=torch.bfloat16)  # A stored transposed
    bt = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    ref = at.float().t() @ bt.float()
    ops.set_mn_major_operands(True)
    try:
        out = ops.gemm_nt(ops.as_operand(at, "columnwise"), ops.as_operand(bt, "columnwise"), out_dtype=torch.float32)
        te.check_status()
    finally:
        ops.set_mn_major_operands(False)
    assert _rel(out, ref) < 1e-3


@pytest.mark.parametrize("R,C", [(128, 128), (256, 384), (160, 96), (1024, 4096)])
@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_quantize_mxfp8_bit_exact(R, C, fp8):
    x = (torch.randn(R, C, device=DEV) * torch.exp(torch.randn(R, 1, device=DEV) * 2)).to(torch.bfloat16)
    rd, rs, cd, cs = qz.quantize_mxfp8(x, fp8)
    rd_r, rs_r, cd_r, cs_r = qz.quantize_mxfp8(x.cpu(), fp8)
    assert torch.equal(rd.cpu(), rd_r)
    assert torch.equal(cd.cpu(), cd_r)
    assert torch.equal(qz.unswizzle_scales(rs, R, C // 32).cpu(), Q.unswizzle_scales(rs_r, R, C // 32))
    assert torch.equal(qz.unswizzle_scales(cs, C, R // 32).cpu(), Q.unswizzle_scales(cs_r, C, R // 32))
    deq = qz.dequantize_mxfp8(rd, rs, fp8, torch.float32)
    deq_r = qz.dequantize_mxfp8(rd_r, rs_r, fp8, torch.float32)
    assert torch.equal(deq.cpu(), deq_r)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (384, 128, 256), (1024, 2048, 4096), (160, 96, 64)])
def test_gemm_mxfp8(M, N, K):
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    qa = MXFP8Quantizer(torch.float8_e4m3fn, columnwise=False)(a)
    qb = MXFP8Quantizer(torch.float8_e4m3fn, columnwise=False)(b)
    ref = qa.dequantize(dtype=torch.float32) @ qb.dequantize(dtype=torch.float32).t()
    out = ops.gemm_nt(ops.as_operand(qa), ops.as_operand(qb), out_dtype=torch.float32)
    te.check_status()
    assert _rel(out, ref) < 1e-4
    # columnwise (transposed) copies give the transposed-operand product
    qa2 = MXFP8Quantizer(torch.float8_e5m2)(a)
    ref2 = qa2.dequantize(dtype=torch.float32)
    got2 = qz.dequantize_mxfp8(qa2._columnwise_data, qa2._columnwise_scale_inv, torch.float8_e5m2, torch.float32)
    assert _rel(got2.t(), a.float()) < 0.1 and ref2.shape == a.shape


def test_quantize_fp8_tensor():
    x = torch.randn(256, 512, device=DEV, dtype=torch.bfloat16)
    scale = torch.full((1,), 3.0, device=DEV)
    amax = torch.zeros(1, device=DEV)
    q = Float8Quantizer(scale, amax, torch.float8_e4m3fn)(x)
    ref = Q.quantize_fp8_tensor(x.cpu(), torch.tensor([3.0]), torch.float8_e4m3fn)
    assert torch.equal(q._data.cpu(), ref.view(torch.uint8))
    assert torch.equal(q._transpose.cpu(), ref.t().contiguous().view(torch.uint8))
    assert abs(amax.item() - x.abs().max().item()) < 1e-6
    qc = Float8CurrentScalingQuantizer(torch.float8_e4m3fn, device=DEV)(x)
    assert _rel(qc.dequantize(dtype=torch.float32), x) < 0.05


@pytest.mark.parametrize("layernorm", [False, True])
@pytest.mark.parametrize("zc", [False, True])
def test_norm_fwd_bwd(layernorm, zc):
    R, C = 512, 1024
    x = torch.randn(R, C, device=DEV, dtype=torch.bfloat16)
    g = (torch.randn(C, device=DEV) * 0.1 + (0 if zc else 1)).to(torch.bfloat16)
    b = torch.randn(C, device=DEV).to(torch.bfloat16) if layernorm else None
    y, _, mu, rs = ops.norm_fwd(x, g, b, 1e-5, zc, layernorm)
    yr, mur, rsr = ops.norm.norm_fwd_ref(x, g, b, 1e-5, zc, layernorm)
    assert _rel(y, yr) < 5e-3 and _rel(rs, rsr) < 1e-5
    dy = torch.randn(R, C, device=DEV, dtype=torch.bfloat16)
    dx, dg, db = ops.norm_bwd(dy, x, mu, rs, g, zc, layernorm)
    dxr, dgr, dbr = ops.norm.norm_bwd_ref(dy, x, mur, rsr, g, zc, layernorm)
    assert _rel(dx, dxr) < 5e-3 and _rel(dg, dgr) < 1e-2
    if layernorm:
        assert _rel(db, dbr) < 1e-2
    # fused MXFP8 output equals quantizing the 16-bit output
    quant = MXFP8Quantizer()
    _, yq, _, _ = ops.norm_fwd(x, g, b, 1e-5, zc, layernorm, quantizer=quant, want_hp=False)
    y2 = quant(y)
    assert torch.equal(yq._rowwise_data, y2._rowwise_data) or _rel(yq.dequantize(), y2.dequantize()) < 2e-2


@pytest.mark.parametrize("name", ["gelu", "silu", "relu", "swiglu", "geglu", "qgelu", "srelu"])
def test_activation(name):
    R, C = 256, 512
    x = torch.randn(R, C, device=DEV, dtype=torch.bfloat16)
    y, _ = ops.activation_fwd(x, name)
    yr = ops.activation.activation_fwd_ref(x, name)
    assert _rel(y, yr) < 5e-3
    dy = torch.randn_like(y)
    dx, _, _ = ops.activation_bwd(dy, x, name)
    dxr = ops.activation.activation_bwd_ref(dy, x, name)
    assert _rel(dx, dxr) < 5e-3
    quant = MXFP8Quantizer()
    _, yq = ops.activation_fwd(x, name, quantizer=quant, want_hp=False)
    assert _rel(yq.dequantize(dtype=torch.float32), yr) < 0.05


def test_multi_tensor_adam_matches_torch():
    ps = [torch.randn(n, device=DEV) for n in (1000, 70000, 3, 1 << 20)]
    gs = [torch.randn_like(p) for p in ps]
    ref_p = [p.clone().requires_grad_(True) for p in ps]
    opt = torch.optim.AdamW(ref_p, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    master = [p.clone() for p in ps]
    model = [p.to(torch.bfloat16) for p in ps]
    m = [torch.zeros_like(p) for p in ps]
    v = [torch.zeros_like(p) for p in ps]
    for step in (1, 2, 3):
        for rp, g in zip(ref_p, gs):
            rp.grad = g.clone()
        opt.step()
        ops.multi_tensor_adam([[g.to(torch.bfloat16).float() for g in gs] if False else gs, model, m, v, master], 1e-2, 0.9, 0.95,
                              1e-8, step, True, True, 0.1)
    for rp, mp, bp in zip(ref_p, master, model):
        assert _rel(mp, rp) < 1e-5
        assert _rel(bp, rp) < 1e-2


def test_cross_entropy():
    R, V = 64, 32000
    logits = torch.randn(R, V, device=DEV, dtype=torch.bfloat16)
    tgt = torch.randint(0, V, (R,), device=DEV)
    tgt[3] = -100
    ref = logits.float().clone().requires_grad_(True)
    lref = torch.nn.functional.cross_entropy(ref, tgt, reduction="none", ignore_index=-100)
    lref.sum().backward()
    loss, grad = ops.cross_entropy_fwd_bwd(logits.clone(), tgt, 1.0, inplace_grad=False)
    assert _rel(loss, lref) < 1e-4
    assert _rel(grad, ref.grad) < 2e-2


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope(interleaved):
    s, b, h, d = 128, 2, 4, 64
    x = torch.randn(s, b, h, d, device=DEV, dtype=torch.bfloat16)
    f = ops.rope_freqs(torch.arange(s, device=DEV), d, 10000.0, interleaved)
    y = ops.rope_apply(x, f, interleaved=interleaved)
    yr = ops.misc.rope_ref(x, f, d, interleaved)
    assert _rel(y, yr) < 1e-2
    g = ops.rope_apply(y, f, interleaved=interleaved, backward=True)
    assert _rel(g, x) < 2e-2  # the rotation is orthogonal: backward undoes forward


@pytest.mark.gpu
@pytest.mark.parametrize("dtypes", [("e4m3", "e4m3"), ("e5m2", "e4m3")])
def test_fp8_per_tensor_gemm_matches_dequantized_matmul(dtypes):
    import transformerengine_b200 as te
    from transformerengine_b200 import ops
    from transformerengine_b200.tensor.float8 import Float8CurrentScalingQuantizer

    torch.manual_seed(0)
    M, N, K = 384, 640, 512
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.1
    dt = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
    qa = Float8CurrentScalingQuantizer(dt[dtypes[0]], device="cuda")(a)
    qb = Float8CurrentScalingQuantizer(dt[dtypes[1]], device="cuda")(b)
    out = ops.gemm_nt(ops.as_operand(qa), ops.as_operand(qb), out_dtype=torch.float32)
    te.ops.check_status()
    ref = qa.dequantize().float() @ qb.dequantize().float().t()
    err = (out - ref).abs().max().item() / ref.abs().max().item()
    assert err < 5e-3, err


@pytest.mark.gpu
@pytest.mark.parametrize("recipe_name", ["DelayedScaling", "Float8CurrentScaling", "Float8BlockScaling"])
def test_linear_under_fp8_recipes_on_gpu(recipe_name):
    import transformerengine_b200 as te

    torch.manual_seed(1)
    lin = te.Linear(512, 768, bias=True, params_dtype=torch.bfloat16, device="cuda")
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    recipe = getattr(te.recipe, recipe_name)()
    for _ in range(2):  # the second pass of delayed scaling uses the recorded amax
        with te.autocast(enabled=True, recipe=recipe):
            y = lin(x)
        y.float().square().mean().backward()
    te.ops.check_status()
    ref = x.detach().float() @ lin.weight.detach().float().t() + lin.bias.detach().float()
    rel = (y.float() - ref).norm() / ref.norm()
    assert rel < 0.08, rel.item()
    assert torch.isfinite(x.grad.float()).all() and torch.isfinite(lin.weight.grad.float()).all()


@pytest.mark.gpu
def test_softmax_and_dropout_kernels():
    from transformerengine_b200.ops import misc

    torch.manual_seed(0)
    b, h, sq, sk = 2, 3, 40, 72
    s = torch.randn(b, h, sq, sk, device="cuda", dtype=torch.bfloat16)
    mask = torch.rand(b, 1, sq, sk, device="cuda") < 0.2
    for causal in (False, True):
        p = misc.scaled_masked_softmax(s, mask, 0.7, causal)
        ref = misc.scaled_masked_softmax(s.cpu(), mask.cpu(), 0.7, causal)
        assert torch.allclose(p.cpu().float(), ref.float(), atol=1e-2)
    dp = torch.randn_like(p)
    dx = misc.softmax_bwd(p, dp, 0.7)
    assert torch.allclose(dx.cpu().float(), misc.softmax_bwd(p.cpu(), dp.cpu(), 0.7).float(), atol=2e-2)
    x = torch.randn(1000, 37, device="cuda", dtype=torch.bfloat16)
    y, keep = misc.dropout_fwd(x, 0.25)
    frac = (y != 0).float().mean().item()
    assert 0.70 < frac < 0.80
    kept = y != 0
    assert torch.allclose(y[kept].float(), x[kept].float() / 0.75, rtol=1e-2)
    g = misc.dropout_bwd(torch.ones_like(x), keep, 0.25)
    nz = x != 0
    assert torch.equal((g != 0)[nz], kept[nz])


@pytest.mark.gpu
@pytest.mark.parametrize("algo", ["max", "most_recent"])
def test_delayed_scaling_update_kernel_matches_reference(algo):
    import transformerengine_b200 as te
    from transformerengine_b200.quantization import RecipeState, update_delayed_scaling_state

    torch.manual_seed(0)
    recipe = te.recipe.DelayedScaling(amax_history_len=8, amax_compute_algo=algo, margin=1)
    st = RecipeState.create(recipe, mode="forward", num_quantizers=6, device=torch.device("cuda"))
    ref = RecipeState.create(recipe, mode="forward", num_quantizers=6, device=torch.device("cpu"))
    h = torch.rand(8, 6) * 10
    h[:, 2] = 0
    st.amax_history.copy_(h)
    ref.amax_history.copy_(h)
    update_delayed_scaling_state(st)
    update_delayed_scaling_state(ref)
    assert torch.allclose(st.scale.cpu(), ref.scale, rtol=1e-6)
    assert torch.equal(st.amax_history.cpu(), ref.amax_history)


@pytest.mark.parametrize("dim", [1, 2])
@pytest.mark.parametrize("R,C", [(256, 384), (300, 160), (128, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fp8_block128_quantizer_matches_reference(dim, R, C, dtype):
    from transformerengine_b200.tensor.blockwise import Float8BlockQuantizer

    x = (torch.randn(R, C, device=DEV) * torch.logspace(-3, 2, C, device=DEV)).to(dtype)
    q = Float8BlockQuantizer(torch.float8_e4m3fn, rowwise=True, columnwise=True, block_scaling_dim=dim)
    got = q(x)
    dims = (128, 128) if dim == 2 else (1, 128)
    rq, rs = Q.quantize_fp8_blockwise(x, torch.float8_e4m3fn, dims, True, 0.0)
    cq, cs = Q.quantize_fp8_blockwise(x.t().contiguous(), torch.float8_e4m3fn, dims, True, 0.0)
    assert torch.equal(got._rowwise_data.view(torch.uint8), rq.view(torch.uint8))
    assert torch.equal(got._columnwise_data.view(torch.uint8), cq.view(torch.uint8))
    assert torch.equal(got._rowwise_scale_inv, rs) and torch.equal(got._columnwise_scale_inv, cs)
    assert _rel(got.dequantize(dtype=torch.float32), x) < 0.05
    # the UE8M0 tiles hold the same scales: block scale of (row i, 128-block kb) repeated four times
    if C % 32 == 0:
        mx = Q.unswizzle_scales(got._rowwise_mx_scale, R, ((C + 127) // 128) * 4)
        want = rs.repeat_interleave(128, 0)[:R] if dim == 2 else rs
        assert torch.equal(torch.exp2(mx.float() - 127.0)[:, ::4], want)


def test_fp8_block_scaled_gemm_runs_on_the_block_scaled_tensor_core_path():
    """1 x 128 activations times 128 x 128 weights: exact product of the dequantized operands."""
    from transformerengine_b200.tensor.blockwise import Float8BlockQuantizer

    M, N, K = 512, 768, 1024
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    qa = Float8BlockQuantizer(torch.float8_e4m3fn, block_scaling_dim=1)(a)
    qw = Float8BlockQuantizer(torch.float8_e4m3fn, block_scaling_dim=2)(w)
    oa, ow = ops.as_operand(qa, "rowwise"), ops.as_operand(qw, "rowwise")
    assert oa.kind == "mxfp8" and ow.kind == "mxfp8"
    out = ops.gemm_nt(oa, ow, out_dtype=torch.float32)
    te.check_status()
    ref = qa.dequantize(dtype=torch.float32) @ qw.dequantize(dtype=torch.float32).t()
    assert _rel(out, ref) < 1e-5
    # wgrad-style product through the column-wise copies
    g = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    qg = Float8BlockQuantizer(torch.float8_e5m2, block_scaling_dim=1)(g)
    dw = ops.gemm_nt(ops.as_operand(qg, "columnwise"), ops.as_operand(qa, "columnwise"), out_dtype=torch.float32)
    refw = Q.dequantize_fp8_blockwise(qg._columnwise_data.view(torch.float8_e5m2), qg._columnwise_scale_inv, (1, 128),
                                      torch.float32) @ \
        Q.dequantize_fp8_blockwise(qa._columnwise_data.view(torch.float8_e4m3fn), qa._columnwise_scale_inv, (1, 128),
                                   torch.float32).t()
    assert _rel(dw, refw) < 1e-5


@pytest.mark.gpu
def test_helper_kernels_match_torch():
    """column_sum, splits_to_offsets, repad_rows, pad_last_dim against plain torch."""
    import torch
    from transformerengine_b200 import ops

    torch.manual_seed(0)
    for R, C, dt in ((8192, 4096, torch.bfloat16), (1000, 264, torch.float16), (65, 4104, torch.float32)):
        x = torch.randn(R, C, device="cuda", dtype=dt)
        got = ops.column_sum(x, torch.float32)
        torch.testing.assert_close(got, x.float().sum(0), rtol=1e-4, atol=1e-2)
        assert torch.equal(got, ops.column_sum(x, torch.float32))          # deterministic
    xs = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)[:, 128:640]   # row stride != width
    torch.testing.assert_close(ops.column_sum(xs, torch.bfloat16).float(), xs.float().sum(0), rtol=2e-2, atol=0.3)
    for n in (1, 8, 300, 2500):
        s = torch.randint(0, 1000, (n,), device="cuda", dtype=torch.int64)
        ref = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(s, 0)]) * 3
        assert torch.equal(ops.splits_to_offsets(s, 3, torch.int64), ref)
        assert torch.equal(ops.splits_to_offsets(s.int(), 3, torch.int32), ref.int())
    m = [37, 0, 128, 5, 1000]
    p = [(v + 127) // 128 * 128 for v in m]
    rows = torch.randn(sum(m), 512, device="cuda", dtype=torch.bfloat16)
    padded = ops.repad_rows(rows, m, p)
    ref = torch.cat([torch.nn.functional.pad(c, (0, 0, 0, pp - mm)) for c, mm, pp in zip(torch.split(rows, m), m, p)])
    assert torch.equal(padded, ref)
    assert torch.equal(ops.repad_rows(padded, p, m), rows)
    mt, pt = torch.tensor(m, device="cuda", dtype=torch.int32), torch.tensor(p, device="cuda", dtype=torch.int32)
    assert torch.equal(ops.repad_rows(rows, mt, pt), ref)                   # splits given on the device
    h = torch.randn(4, 16, 8, 72, device="cuda", dtype=torch.bfloat16)
    hp = ops.pad_last_dim(h, 128)
    assert hp.shape == (4, 16, 8, 128) and torch.equal(hp[..., :72], h) and hp[..., 72:].abs().sum() == 0
    assert torch.equal(ops.pad_last_dim(hp, 72), h)


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["grouped", "blocked"])
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_packed_qkv_one_launch(layout, interleaved):
    """Query and key heads of a packed QKV tensor rotated by ONE kernel (in place and out of place, forward and
    backward, separate key angles) against the plain rotation of the split views."""
    import torch
    from transformerengine_b200 import ops

    torch.manual_seed(1)
    s, b, hq, hk, d = 96, 2, 8, 2, 128
    g = hq // hk
    x = torch.randn(s, b, hq + 2 * hk, d, device="cuda", dtype=torch.bfloat16)
    fq = ops.rope_freqs(torch.arange(s, device="cuda"), d, 10000.0, interleaved)
    fk = ops.rope_freqs(torch.arange(s, device="cuda"), d, 500000.0, interleaved)

    def split(t):
        if layout == "grouped":
            t5 = t.unflatten(2, (hk, g + 2))
            return t5[:, :, :, :g].reshape(s, b, hq, d), t5[:, :, :, g], t5[:, :, :, g + 1]
        return t[:, :, :hq], t[:, :, hq:hq + hk], t[:, :, hq + hk:]

    for backward in (False, True):
        y = ops.rope_qkv(x, fq, fk, layout=layout, hq=hq, hk=hk, interleaved=interleaved, backward=backward)
        q, k, v = split(x)
        yq, yk, yv = split(y)
        assert torch.equal(yq, ops.rope_apply(q.contiguous(), fq, interleaved=interleaved, backward=backward))
        assert torch.equal(yk, ops.rope_apply(k.contiguous(), fk, interleaved=interleaved, backward=backward))
        assert torch.equal(yv, v)
    z = x.clone()
    ops.rope_qkv(z, fq, fk, layout=layout, hq=hq, hk=hk, interleaved=interleaved, inplace=True)
    assert torch.equal(z, ops.rope_qkv(x, fq, fk, layout=layout, hq=hq, hk=hk, interleaved=interleaved))
    # the strided [s, b, h, d] view of a batch-first tensor
    xb = x.transpose(0, 1).contiguous()
    yb = ops.rope_qkv(xb.transpose(0, 1), fq, fq, layout=layout, hq=hq, hk=hk, interleaved=interleaved)
    assert torch.equal(yb, ops.rope_qkv(x, fq, fq, layout=layout, hq=hq, hk=hk, interleaved=interleaved))


@pytest.mark.gpu
def test_grouped_sums_bias_add_and_row_dot():
    import torch
    from transformerengine_b200 import ops

    torch.manual_seed(2)
    m = [300, 0, 1029, 7]
    offs = torch.tensor([0, 300, 300, 1329, 1336], dtype=torch.int32, device="cuda")
    for dt in (torch.bfloat16, torch.float32):
        x = torch.randn(sum(m), 520, device="cuda", dtype=dt)
        got = ops.grouped_column_sum(x, offs, torch.float32)
        ref = torch.stack([c.float().sum(0) for c in torch.split(x, m)])
        torch.testing.assert_close(got, ref, rtol=1e-4, atol=2e-2)
        bias = torch.randn(4, 520, device="cuda", dtype=dt)
        y = x.clone()
        ops.grouped_bias_add_(y, bias, offs)
        refy = torch.cat([c + bias[g] for g, c in enumerate(torch.split(x, m))])
        torch.testing.assert_close(y, refy)
        a, b = torch.randn(777, 1032, device="cuda", dtype=dt), torch.randn(777, 1032, device="cuda", dtype=dt)
        torch.testing.assert_close(ops.row_dot(a, b), (a.float() * b.float()).sum(-1), rtol=1e-4, atol=1e-2)


@pytest.mark.gpu
def test_kernels_stay_inside_their_outputs():
    """Guard bands around every output that the Python wrappers allocate: quantizers with swizzled scale layouts
    on shapes with partial tiles, GEMMs with TMA-store epilogues on ragged widths, strided RoPE, norm."""
    import torch
    from transformerengine_b200 import ops
    from transformerengine_b200.ops import quantize as qz
    from transformerengine_b200.tensor import MXFP8Quantizer
    from transformerengine_b200.utils.canary import GuardedAllocation

    torch.manual_seed(5)
    g = GuardedAllocation()
    x = torch.randn(1040, 272, device="cuda", dtype=torch.bfloat16)
    a = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(264, 512, device="cuda", dtype=torch.bfloat16)
    xq = torch.randn(384, 640, device="cuda", dtype=torch.bfloat16)
    with g.intercept():
        qz.quantize_nvfp4(x, with_rht=True)                       # one-pass kernel, partial tiles
        qz.quantize_nvfp4(x, rowwise=True, columnwise=False)
        qz.quantize_mxfp8(xq, torch.float8_e4m3fn)                # tile quantizer, swizzled scales
        ops.gemm_nt(a, b, out_dtype=torch.bfloat16)               # ragged M and N
        qa, qb = MXFP8Quantizer(columnwise=False)(a[:256]), MXFP8Quantizer(columnwise=False)(b[:256])   # whole 128-row scale tiles
        ops.gemm_nt(ops.as_operand(qa), ops.as_operand(qb), out_dtype=torch.bfloat16)
        ops.column_sum(a, torch.float32)
        ops.norm_fwd(a, torch.ones(512, device="cuda", dtype=torch.bfloat16), None, 1e-5, False, False)
        f = ops.rope_freqs(torch.arange(96, device="cuda"), 128, 10000.0, False)
        ops.rope_qkv(torch.randn(96, 2, 12, 128, device="cuda", dtype=torch.bfloat16), f, f, layout="grouped", hq=8, hk=2)
    torch.cuda.synchronize()
    assert len(g._allocs) >= 8
    g.check()
