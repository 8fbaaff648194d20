"""Numerics of the pure-PyTorch quantization path (the oracle of the CUDA kernels)."""
import pickle

import pytest
import torch

import transformerengine_b200 as te
from transformerengine_b200.ops.ref import quant as Q
from transformerengine_b200.tensor import (Float8BlockQuantizer, Float8CurrentScalingQuantizer, Float8Quantizer,
                                           MXFP8Quantizer, NVFP4Quantizer)


def test_float_to_e8m0_rounds_up_and_saturates():
    v = torch.tensor([0.0, 1.0, 1.0001, 0.5, 3.0, float("inf"), float("nan"), 2.0 ** -127, 2.0 ** -126 * 0.75])
    e = Q.float_to_e8m0(v)
    assert e.tolist()[:5] == [0, 127, 128, 126, 129]
    assert e[5].item() == 0xFE and e[6].item() == 0xFF
    assert e[7].item() == 0  # 2^-127 is representable as exponent 0
    assert e[8].item() == 1  # above 2^-127: rounds up to 2^-126
    back = Q.e8m0_to_float(e[:5])
    assert torch.all(back >= v[:5])


def test_mxfp8_quantize_roundtrip_and_scale_rule():
    x = torch.randn(64, 128) * torch.exp(torch.randn(64, 1) * 3)
    q, e = Q.quantize_mxfp8_rowwise(x, torch.float8_e4m3fn)
    amax = x.reshape(64, 4, 32).abs().amax(-1)
    scale = Q.e8m0_to_float(e)
    # scaled block maximum fits the format, and the scale is the smallest power of two that does
    assert torch.all(amax / scale <= 448.0)
    assert torch.all((amax / (scale / 2) > 448.0) | (amax == 0))
    deq = Q.dequantize_mxfp8_rowwise(q, e, torch.float32)
    assert ((deq - x).abs() <= x.reshape(64, 4, 32).abs().amax(-1).repeat_interleave(32, 1) * 0.07).all()


def test_swizzle_roundtrip_and_index_formula():
    R, K = 200, 10
    e = torch.randint(0, 255, (R, K), dtype=torch.uint8)
    s = Q.swizzle_scales(e)
    assert torch.equal(Q.unswizzle_scales(s, R, K), e)
    kt = (K + 3) // 4
    for i, j in [(0, 0), (33, 1), (130, 5), (199, 9)]:
        off = ((i // 128) * kt + j // 4) * 512 + (i % 32) * 16 + ((i % 128) // 32) * 4 + j % 4
        assert s[off] == e[i, j]


def test_fp8_scale_rule():
    amax = torch.tensor([0.0, 1.0, float("inf"), 448.0])
    prev = torch.tensor([3.0, 3.0, 3.0, 3.0])
    s = Q.compute_scale_from_amax(amax, 448.0, margin=1, prev_scale=prev)
    assert s.tolist() == [3.0, 224.0, 3.0, 0.5]
    p2 = Q.compute_scale_from_amax(torch.tensor([3.0]), 448.0, force_pow_2=True)
    assert p2.item() == 128.0  # 448/3 = 149.3 floors to 2^7


def test_nvfp4_codes_round_to_nearest_even():
    x = torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -0.3, -6.0, 0.0, 0.26, 5.01, -2.5, 1.0]])
    c = Q.cast_to_e2m1_codes(x)[0].tolist()
    assert c == [0, 2, 2, 4, 4, 6, 6, 7, 8, 9, 15, 0, 1, 7, 12, 2]


def test_nvfp4_quantize_dequantize_error():
    x = torch.randn(128, 256)
    amax = Q.amax_abs(x)
    d, s = Q.quantize_nvfp4_1d(x, amax)
    deq = Q.dequantize_nvfp4(d, s, amax, torch.float32)
    rel = (deq - x).norm() / x.norm()
    assert rel < 0.15
    d2, s2 = Q.quantize_nvfp4_2d(x, amax)
    # 2-D scales: the transposed quantization sees the same block scales
    d2t, s2t = Q.quantize_nvfp4_2d(x.t().contiguous(), amax)
    a = Q.dequantize_nvfp4(d2, s2, amax, torch.float32)
    b = Q.dequantize_nvfp4(d2t, s2t, amax, torch.float32).t()
    assert torch.equal(a, b)


def test_rht_is_orthogonal_and_sr_is_unbiased():
    h = Q.hadamard_matrix_16()
    assert torch.allclose(h @ h.t(), torch.eye(16), atol=1e-6)
    x = torch.full((64, 64), 0.7)
    g = torch.Generator().manual_seed(0)
    acc = torch.zeros_like(x)
    for _ in range(64):
        codes = Q.stochastic_round_e2m1_codes(x, torch.rand(x.shape, generator=g))
        acc += Q.e2m1_codes_to_float(codes)
    assert abs((acc / 64).mean().item() - 0.7) < 0.01  # round-to-nearest would give 0.5 or 1.0


@pytest.mark.parametrize("make", [
    lambda: Float8Quantizer(torch.ones(1), torch.zeros(1), torch.float8_e4m3fn),
    lambda: Float8CurrentScalingQuantizer(torch.float8_e4m3fn),
    lambda: MXFP8Quantizer(),
    lambda: NVFP4Quantizer(),
    lambda: NVFP4Quantizer(with_rht=True),
    lambda: Float8BlockQuantizer(block_scaling_dim=1),
    lambda: Float8BlockQuantizer(block_scaling_dim=2),
])
def test_quantized_tensor_behaviour(make):
    q = make()
    x = torch.randn(128, 256)
    t = q(x)
    assert isinstance(t, te.tensor.QuantizedTensor) and t.shape == x.shape
    tol = 0.2 if isinstance(q, NVFP4Quantizer) else 0.08
    assert (t.dequantize() - x).norm() / x.norm() < tol
    # columnwise copy alone dequantizes to the same logical tensor
    t2 = t.detach()
    t2.update_usage(rowwise_usage=False)
    assert (t2.dequantize() - x).norm() / x.norm() < tol
    # generic torch ops see dequantized values; pickling keeps the payload
    assert torch.allclose((t + 1).float(), t.dequantize().float() + 1)
    r = pickle.loads(pickle.dumps(t))
    assert torch.equal(r.dequantize(), t.dequantize())
    # in-place update re-quantizes
    t.copy_(torch.zeros_like(x))
    assert t.dequantize().abs().max() == 0


def test_make_empty_and_update_quantized():
    q = MXFP8Quantizer()
    t = q.make_empty((64, 64), dtype=torch.bfloat16)
    x = torch.randn(64, 64)
    q.update_quantized(x, t)
    assert torch.equal(t.dequantize(dtype=torch.float32), q(x).dequantize(dtype=torch.float32))


def test_standalone_hadamard_transform_matches_the_quantizer():
    import torch
    from transformerengine_b200 import ops
    from transformerengine_b200.ops import quantize as qz

    torch.manual_seed(0)
    x = torch.randn(64, 48)
    y = ops.hadamard_transform(x)
    torch.testing.assert_close(y.norm(), x.norm(), rtol=1e-5, atol=1e-5)          # orthogonal
    torch.testing.assert_close(ops.hadamard_transform(x, transposed=True), ops.hadamard_transform(x.t().contiguous()))
    # the quantizer's column-wise amax is the amax of the rotated transpose
    xb = x.to(torch.bfloat16)
    res = qz.quantize_nvfp4(xb, with_rht=True)
    want = ops.hadamard_transform(xb.float(), transposed=True).abs().max()
    torch.testing.assert_close(res[5].reshape(()).float(), want, rtol=1e-6, atol=0)


def test_quantizer_and_tensor_conveniences():
    """Small API of the quantizers / quantized tensors: shapes of the scale buffers and the column-wise copy,
    determinism flags, wrapping existing bytes, metadata, make_like, clear, copy_from_storage."""
    import transformerengine_b200 as te
    from transformerengine_b200.tensor.blockwise import Float8BlockQuantizer
    from transformerengine_b200.tensor.float8 import Float8CurrentScalingQuantizer, Float8Quantizer
    from transformerengine_b200.tensor.mxfp8 import MXFP8Quantizer
    from transformerengine_b200.tensor.nvfp4 import NVFP4Quantizer

    x = torch.randn(64, 96)
    mx = MXFP8Quantizer()
    q = mx(x)
    assert mx.get_scale_shape(x.shape, False) == (128, 4) and q._rowwise_scale_inv.numel() == 128 * 4
    assert mx.get_scale_shape(x.shape, True) == (128, 4) and mx.get_columnwise_shape(x.shape) == (96, 64)
    assert tuple(q._columnwise_data.shape) == mx.get_columnwise_shape(x.shape)
    nv = NVFP4Quantizer()
    n = nv(x)
    assert nv.get_scale_shape(x.shape, False) == (128, 8) and n._rowwise_scale_inv.numel() == 128 * 8
    assert nv.convert_shape_for_fp4((64, 96)) == (64, 48) == tuple(n._rowwise_data.shape)
    blk = Float8BlockQuantizer(block_scaling_dim=2)
    assert blk.get_scale_shape((300, 200), False) == (3, 2) and blk.get_scale_shape((300, 200), True) == (2, 3)
    assert Float8BlockQuantizer(block_scaling_dim=1).get_scale_shape((300, 200), False) == (300, 2)
    cur = Float8CurrentScalingQuantizer(torch.float8_e4m3fn)
    delayed = Float8Quantizer(torch.ones(1), torch.zeros(1), torch.float8_e4m3fn)
    assert [z.is_requantization_safe() for z in (mx, nv, blk, cur, delayed)] == [True, True, True, True, False]
    assert not NVFP4Quantizer(stochastic_rounding=True).is_requantization_safe()
    assert te.HybridQuantizer(rowwise_quantizer=MXFP8Quantizer(),
                              columnwise_quantizer=Float8CurrentScalingQuantizer(torch.float8_e4m3fn)).is_requantization_safe()
    a, b = mx.multi_quantize([x, 2 * x])
    assert torch.equal(a.dequantize() * 2, b.dequantize())
    # wrapping bytes that already exist
    back = mx.create_tensor_from_data(q._rowwise_data, q._rowwise_scale_inv, fake_dtype=torch.float32)
    assert torch.equal(back.dequantize(), q.dequantize())
    c = cur(x)
    again = cur.create_tensor_from_data(c._data, scale_inv=c._scale_inv)
    assert torch.equal(again.dequantize(), c.dequantize())
    # current scaling with an amax the caller already has; scale / amax outputs
    amax, scale = x.abs().amax().reshape(1).clone(), torch.zeros(1)
    pre = Float8CurrentScalingQuantizer(torch.float8_e4m3fn, use_existing_amax=True, amax=amax, scale=scale)
    assert torch.equal(pre(x).dequantize(), c.dequantize()) and float(scale) > 0
    # tensor conveniences
    meta = c.get_metadata()
    rebuilt = type(c)(shape=c.shape, dtype=c.dtype, **meta)
    assert torch.equal(rebuilt.dequantize(), c.dequantize())
    like = type(c).make_like(c, dtype=torch.bfloat16, requires_grad=True)
    assert like.dtype == torch.bfloat16 and like.requires_grad and like._data is c._data
    c.update_usage(columnwise_usage=True)
    assert c._transpose is not None
    c.remove_caches()
    assert c._transpose is None
    dst = mx.make_empty(x.shape)
    dst.copy_from_storage(q)
    assert torch.equal(dst.dequantize(), q.dequantize())
    with pytest.raises(ValueError):
        mx.make_empty((32, 96)).copy_from_storage(q)
    q.update_quantizer(MXFP8Quantizer(rowwise=True, columnwise=False))
    with pytest.raises(TypeError):
        q.update_quantizer(cur)
    q.clear()
    assert q._rowwise_data.numel() == 0
    h = te.HybridQuantizer(rowwise_quantizer=Float8CurrentScalingQuantizer(torch.float8_e4m3fn),
                           columnwise_quantizer=MXFP8Quantizer())
    assert not h.with_amax_reduction and h.amax_reduction_group is None
    h.with_amax_reduction = True
    assert h.rowwise_quantizer.with_amax_reduction


@pytest.mark.parametrize("mode", ["MAE", "MSE"])
def test_nvfp4_four_over_six_never_loses_to_standard_scaling(mode):
    """Adaptive block scaling keeps, per 16-value block, the better of map-to-6 and map-to-4: against the standard
    quantization with the same tensor scale no block gets a larger error, some get a smaller one, and the chosen
    block scales are either the standard ones or 1.5 x larger."""
    from transformerengine_b200.ops import quantize as OQ
    from transformerengine_b200.ops.ref import quant as Q
    torch.manual_seed(0)
    x = (torch.randn(64, 128) * torch.rand(64, 1) * 3).to(torch.bfloat16).float()
    rd6, rs6, ar6, *_ = OQ.quantize_nvfp4(x, columnwise=False, e4m3_max=256.0)
    rd, rs, ar, *_ = OQ.quantize_nvfp4(x, columnwise=False, four_over_six=mode, e4m3_max=256.0)
    assert torch.equal(ar, ar6) and torch.allclose(ar, x.abs().amax() * 448 / 256)
    d6 = OQ.dequantize_nvfp4(rd6, rs6, ar6, 64, 128, torch.float32)
    d = OQ.dequantize_nvfp4(rd, rs, ar, 64, 128, torch.float32)
    metric = (lambda e: e.abs()) if mode == "MAE" else (lambda e: e.square())
    e6 = metric(d6 - x).reshape(64, 8, 16).sum(-1)
    e = metric(d - x).reshape(64, 8, 16).sum(-1)
    assert (e <= e6 + 1e-6).all() and (e < e6 - 1e-6).float().mean() > 0.05
    s6 = Q.unswizzle_scales(rs6, 64, 8).view(torch.float8_e4m3fn).float()
    s = Q.unswizzle_scales(rs, 64, 8).view(torch.float8_e4m3fn).float()
    changed = s != s6
    assert changed.any() and ((s[changed] / s6[changed]) - 1.5).abs().max() < 0.2      # 1.5 x, both rounded to E4M3
    assert (e[changed] < e6[changed]).all()          # map-to-4 is only taken where it wins (ties keep map-to-6)
    with pytest.raises(NotImplementedError):
        OQ.quantize_nvfp4(x, with_rht=True, four_over_six=mode)


def test_nvfp4_four_over_six_recipe_and_quantizer_rebuild_on_recipe_change():
    import transformerengine_b200 as te
    from transformerengine_b200.common import recipe as R
    torch.manual_seed(0)
    lin = te.Linear(128, 128, bias=False, params_dtype=torch.float32, device="cpu")
    x = torch.randn(64, 128) * torch.rand(64, 1) * 3
    want = x @ lin.weight.t()

    def err(rec):
        with te.autocast(enabled=True, recipe=rec), torch.no_grad():
            return float((lin(x) - want).abs().mean())

    plain = err(R.NVFP4BlockScaling(disable_rht=True, disable_stochastic_rounding=True))
    adaptive = err(R.NVFP4BlockScaling(disable_rht=True, disable_stochastic_rounding=True, nvfp4_4over6="all"))
    q = lin.quantizers["scaling_fwd"]
    assert q[0].nvfp4_use_4over6 and q[0].nvfp4_e4m3_max == 256 and q[1].nvfp4_use_4over6
    assert adaptive < plain                       # the same module picked up the new recipe's quantizers
    only_w = R.NVFP4BlockScaling(disable_rht=True, disable_stochastic_rounding=True, nvfp4_4over6="weights",
                                 nvfp4_4over6_e4m3_use_256="none", nvfp4_4over6_err_mode="mse")
    err(only_w)
    q = lin.quantizers["scaling_fwd"]
    assert not q[0].nvfp4_use_4over6 and q[1].nvfp4_use_4over6 and q[1].nvfp4_e4m3_max == 448
    assert q[1].nvfp4_4over6_err_mode == "MSE"
    with pytest.raises(ValueError):
        err(R.NVFP4BlockScaling(nvfp4_4over6="all"))              # needs the transform switched off
    with pytest.raises(NotImplementedError):
        err(R.NVFP4BlockScaling(row_scaled_activation=True))
    with pytest.raises(AssertionError):
        R.NVFP4BlockScaling(nvfp4_4over6="some")


@pytest.mark.parametrize("shape", [(64, 64), (256, 288), (320, 96)])
def test_mxfp8_2d_quantization(shape):
    """32 x 32 block scales: the row-wise scale is constant over the 32 rows of a block, the column-wise copy is
    the transpose of the row-wise one, and the values are those of a per-block reference
    (test model: the reference's ``tests/pytorch/test_mxfp8_2d_quantize.py``)."""
    import transformerengine_b200 as te
    from transformerengine_b200.common import recipe as R
    from transformerengine_b200.ops.ref import quant as Q
    from transformerengine_b200.tensor.mxfp8 import MXFP8Quantizer
    torch.manual_seed(0)
    rows, cols = shape
    x = (torch.randn(rows, cols) * torch.rand(rows, 1) * 4).to(torch.bfloat16).float()
    q = MXFP8Quantizer(with_2d_quantization=True)(x)
    rs = Q.unswizzle_scales(q._rowwise_scale_inv, rows, cols // 32)
    cs = Q.unswizzle_scales(q._columnwise_scale_inv, cols, rows // 32)
    assert torch.equal(rs.reshape(rows // 32, 32, -1), rs[::32][:, None].expand(-1, 32, -1))
    assert torch.equal(cs.reshape(cols // 32, 32, -1), cs[::32][:, None].expand(-1, 32, -1))
    assert torch.equal(rs[::32], cs[::32].t())
    assert torch.equal(q._columnwise_data, q._rowwise_data.reshape(rows, cols).t())
    # per-block reference: scale 2^ceil(log2(amax / 448)), values rounded to E4M3
    blocks = x.reshape(rows // 32, 32, cols // 32, 32)
    amax = blocks.abs().amax(dim=(1, 3))
    scale_inv = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
    want = (blocks / scale_inv[:, None, :, None]).to(torch.float8_e4m3fn).float() * scale_inv[:, None, :, None]
    torch.testing.assert_close(q.dequantize(), want.reshape(rows, cols), rtol=0, atol=0)
    col_only = MXFP8Quantizer(with_2d_quantization=True, rowwise=False)(x)
    torch.testing.assert_close(col_only.dequantize(), q.dequantize(), rtol=0, atol=0)
    if shape == (64, 64):
        lin = te.Linear(64, 64, bias=False, params_dtype=torch.float32, device="cpu")
        with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling(enable_2d_quantization=True)):
            y = lin(x.requires_grad_())
        qs = lin.quantizers["scaling_fwd"]
        assert qs[1].with_2d_quantization and not qs[0].with_2d_quantization
        wd = MXFP8Quantizer(with_2d_quantization=True)(lin.weight.detach()).dequantize()
        xd = MXFP8Quantizer()(x.detach()).dequantize()
        torch.testing.assert_close(y, xd @ wd.t(), rtol=1e-5, atol=1e-5)
        y.sum().backward()
        # dgrad reads the column-wise copy of the weight: with 2-D blocks it is the same matrix
        go = MXFP8Quantizer(torch.float8_e4m3fn)(torch.ones(64, 64)).dequantize()
        torch.testing.assert_close(x.grad, go @ wd, rtol=1e-5, atol=1e-5)
