"""Identity and hybrid quantizers: directions, pickling and use inside a module through a custom recipe
(test model: reference ``tests/pytorch/test_custom_recipe.py``)."""
import io

import torch

import transformerengine_b200 as te
from transformerengine_b200.ops.gemm import as_operand
from transformerengine_b200.tensor import (HybridQuantizedTensor, HybridQuantizer, IdentityQuantizer, IdentityTensor,
                                           MXFP8Quantizer, NVFP4Quantizer)


def test_identity_quantizer_round_trip_and_pickle():
    x = torch.randn(64, 32)
    q = IdentityQuantizer(dtype=torch.bfloat16)
    t = q(x)
    assert isinstance(t, IdentityTensor) and t.shape == x.shape and t.dtype == torch.float32
    torch.testing.assert_close(t.dequantize(), x.bfloat16().float())
    buf = io.BytesIO()
    torch.save(t, buf)
    buf.seek(0)
    u = torch.load(buf, weights_only=False)
    torch.testing.assert_close(u.dequantize(), t.dequantize())
    q.update_quantized(torch.ones(64, 32), t)
    assert t.dequantize().eq(1).all()


def test_hybrid_quantizer_uses_one_child_per_direction():
    torch.manual_seed(0)
    x = torch.randn(128, 64)
    q = HybridQuantizer(rowwise_quantizer=MXFP8Quantizer(torch.float8_e4m3fn), columnwise_quantizer=NVFP4Quantizer())
    t = q(x)
    assert isinstance(t, HybridQuantizedTensor)
    assert as_operand(t, "rowwise").kind == "mxfp8" and as_operand(t, "columnwise").kind == "nvfp4"
    assert t._rowwise.get_usages() == {"rowwise": True, "columnwise": False}
    assert (t.dequantize() - x).abs().max() < 0.3
    t.update_usage(rowwise_usage=False)
    assert t.get_usages() == {"rowwise": False, "columnwise": True}
    # double quantization: the columnwise copy is built from the rounded rowwise values
    q2 = HybridQuantizer(rowwise_quantizer=MXFP8Quantizer(torch.float8_e4m3fn), columnwise_quantizer=IdentityQuantizer(),
                         columnwise_source="rowwise_dequantized")
    t2 = q2(x)
    torch.testing.assert_close(t2._columnwise.dequantize(), t2._rowwise.dequantize(dtype=torch.float32))
    try:
        same = IdentityQuantizer()
        HybridQuantizer(rowwise_quantizer=same, columnwise_quantizer=same)
        raise AssertionError("shared child must be rejected")
    except ValueError:
        pass


def test_linear_with_hybrid_weight_quantizer_in_custom_recipe():
    torch.manual_seed(0)

    def factory(role):
        if role == "linear_weight":
            return HybridQuantizer(rowwise_quantizer=MXFP8Quantizer(torch.float8_e4m3fn),
                                   columnwise_quantizer=IdentityQuantizer(dtype=torch.bfloat16))
        if role in ("linear_input", "linear_grad_output"):
            return MXFP8Quantizer(torch.float8_e4m3fn if role == "linear_input" else torch.float8_e5m2)
        return None

    lin = te.Linear(64, 96, bias=True, params_dtype=torch.float32)
    x = torch.randn(32, 64, requires_grad=True)
    with te.autocast(enabled=True, recipe=te.recipe.CustomRecipe(qfactory=factory)):
        y = lin(x)
    y.sum().backward()
    ref = torch.nn.functional.linear(x, lin.weight, lin.bias)
    assert (y - ref).abs().max() < 0.25 * ref.abs().max()
    assert x.grad is not None and lin.weight.grad is not None
    gref = torch.ones(32, 96) @ lin.weight
    assert (x.grad - gref).abs().max() < 0.1 * gref.abs().max() + 0.05


def test_grouped_tensor_members_share_one_buffer_and_quantize_per_member():
    from transformerengine_b200.tensor import GroupedTensor

    g = GroupedTensor.make_grouped_tensor_with_shapes(3, [(32, 64)] * 3, dtype=torch.bfloat16)
    assert g.all_same_shape() and g.logical_shape == (96, 64) and g.first_dims is None
    ws = [torch.randn(32, 64) for _ in range(3)]
    g.quantize(ws)
    m = g.split_into_quantized_tensors()
    assert m[1].data_ptr() == g.data.data_ptr() + 32 * 64 * 2  # views of the packed buffer
    torch.testing.assert_close(g.stacked()[2].float(), ws[2].bfloat16().float())
    assert g.tensor_offsets.tolist() == [0, 2048, 4096, 6144]

    # ragged members (tokens per expert) with an MXFP8 quantizer
    first = torch.tensor([32, 96, 64])
    gq = GroupedTensor.make_grouped_tensor(3, first, None, 192, 64, quantizer=MXFP8Quantizer(torch.float8_e4m3fn))
    assert not gq.all_same_first_dim() and gq.get_common_last_dim() == 64
    xs = [torch.randn(int(n), 64) for n in first]
    parts = gq.quantize(xs)
    assert gq.has_data() and gq.has_columnwise_data()
    for p, x in zip(parts, xs):
        assert as_operand(p, "rowwise").kind == "mxfp8"
        assert (p.dequantize(dtype=torch.float32) - x).abs().max() < 0.25
    saved, obj = gq.prepare_for_saving()
    assert obj.restore_from_saved(saved) == []
    assert gq.rowwise_data.numel() == 192 * 64

    w = torch.arange(2 * 4 * 8, dtype=torch.float32)
    gw = GroupedTensor.make_grouped_tensor_from_rowwise_data(num_tensors=2, tensor_shape=(4, 8), rowwise_data=w)
    assert gw.split_into_quantized_tensors()[1][0, 0] == 32
