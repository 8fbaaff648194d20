"""Factory zoo: every factory trains a Linear through ``CustomRecipe`` close to the fp32 result."""
import pytest
import torch

import transformerengine_b200 as te
from transformerengine_b200.custom_recipes import custom_gemm, quantizer_factories as qf, quantizer_factory_zoo as zoo
from transformerengine_b200.tensor import MXFP8Quantizer

FACTORIES = [qf.high_precision_factory, qf.identity_factory, qf.current_scaling_factory, qf.float8_block_scaling_factory,
             qf.mxfp8_factory, qf.nvfp4_factory, zoo.mxfp8_fwd_nvfp4_bwd_factory,
             zoo.high_precision_fwd_mxfp8_bwd_factory, zoo.mxfp8_fwd_high_precision_bwd_factory,
             zoo.nvfp4_1d_weight_factory]


@pytest.mark.parametrize("factory", FACTORIES, ids=lambda f: f.__name__)
def test_factory_trains_a_linear(factory):
    torch.manual_seed(0)
    lin = te.Linear(128, 128, bias=False, params_dtype=torch.float32, device="cpu")
    x = torch.randn(64, 128, requires_grad=True)
    with te.autocast(enabled=True, recipe=te.recipe.CustomRecipe(qfactory=factory)):
        y = lin(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref = x.detach() @ lin.weight.detach().t()
    tol = 0.35 if "nvfp4" in factory.__name__ else 0.1
    assert (y - ref).abs().max() < tol * ref.abs().max()
    gx = dy @ lin.weight.detach()
    gw = dy.t() @ x.detach()
    assert (x.grad - gx).abs().max() < tol * gx.abs().max() * 1.5
    assert (lin.weight.grad - gw).abs().max() < tol * gw.abs().max() * 1.5


def test_custom_gemm_layouts_on_quantized_operands():
    torch.manual_seed(0)
    w, x, dy = torch.randn(64, 32), torch.randn(96, 32), torch.randn(96, 64)
    q = MXFP8Quantizer(torch.float8_e4m3fn)
    wq, xq = q(w), q(x)
    wd, xd = wq.dequantize(dtype=torch.float32), xq.dequantize(dtype=torch.float32)
    torch.testing.assert_close(custom_gemm(wq, xq, layout="TN"), xd @ wd.t())
    torch.testing.assert_close(custom_gemm(wq, dy, layout="NN"), dy @ wd)
    torch.testing.assert_close(custom_gemm(xq, dy, layout="NT"), dy.t() @ xd)


def test_delayed_scaling_request_equals_the_delayed_scaling_recipe():
    """A custom recipe whose factory asks for library-managed delayed scaling trains exactly like the DelayedScaling
    recipe with the same parameters (scales follow the amax history, updated at region exit)."""
    from transformerengine_b200.common import recipe as R
    from transformerengine_b200.custom_recipes.quantizer_factories import tensor_type

    def factory(role):
        if tensor_type(role) in ("output", "grad_input"):
            return None
        return te.DelayedScalingRequest(amax_history_len=4, margin=0)

    def run(rec):
        torch.manual_seed(0)
        lin = te.Linear(32, 32, bias=False, params_dtype=torch.float32, device="cpu")
        outs = []
        for step in range(4):
            x = (torch.randn(16, 32) * (step + 1)).requires_grad_()
            with te.autocast(enabled=True, recipe=rec):
                y = lin(x)
            y.square().sum().backward()
            outs.append((y.detach().clone(), x.grad.clone(), lin.weight.grad.clone()))
            lin.weight.grad = None
        return outs

    a = run(R.CustomRecipe(qfactory=factory))
    b = run(R.DelayedScaling(amax_history_len=4, margin=0))
    for (ya, gxa, gwa), (yb, gxb, gwb) in zip(a, b):
        torch.testing.assert_close(ya, yb, rtol=0, atol=0)
        torch.testing.assert_close(gxa, gxb, rtol=0, atol=0)
        torch.testing.assert_close(gwa, gwb, rtol=0, atol=0)


def test_top_level_names_of_the_reference_front_end_exist():
    for name in ("DType", "Float8Quantizer", "MXFP8Tensor", "NVFP4Quantizer", "Float8BlockwiseQTensor",
                 "HybridQuantizer", "IdentityQuantizer", "QuantizedTensor", "Quantizer", "QuantizerRole",
                 "DelayedScalingRequest", "ManualOffloadSynchronizer", "mark_not_offload", "prepare_for_saving",
                 "restore_from_saved", "interleave_glu_tensor", "get_device_compute_capability",
                 "UserBufferQuantizationMode", "constants", "load_framework_extension"):
        assert hasattr(te, name), name
    assert te.DType.kFloat8E4M3 == te.constants.TE_DType[torch.float8_e4m3fn]
    assert str(te.QuantizerRole(module_type="linear", tensor_type="input")) == "module_type=linear|tensor_type=input"


def test_delayed_scaling_requests_as_children_of_a_hybrid_quantizer():
    """Requests may stand in for the children of a ``HybridQuantizer``: the recipe state gives each child its own
    slot of the amax history.  Two delayed children reproduce the DelayedScaling recipe bit for bit; a delayed
    row-wise child next to an MXFP8 column-wise child runs and keeps a history."""
    from transformerengine_b200.common import recipe as R
    from transformerengine_b200.custom_recipes.quantizer_factories import tensor_type
    from transformerengine_b200.tensor.mxfp8 import MXFP8Quantizer

    req = te.DelayedScalingRequest(amax_history_len=4, margin=0)

    def both(role):
        if tensor_type(role) in ("output", "grad_input"):
            return None
        return te.HybridQuantizer(rowwise_quantizer=req, columnwise_quantizer=req)

    def mixed(role):
        if tensor_type(role) in ("output", "grad_input"):
            return None
        return te.HybridQuantizer(rowwise_quantizer=req, columnwise_quantizer=MXFP8Quantizer())

    def run(rec):
        torch.manual_seed(0)
        lin = te.Linear(32, 32, bias=False, params_dtype=torch.float32, device="cpu")
        outs = []
        for step in range(4):
            x = (torch.randn(32, 32) * (step + 1)).requires_grad_()
            with te.autocast(enabled=True, recipe=rec):
                y = lin(x)
            y.square().sum().backward()
            outs.append((y.detach().clone(), x.grad.clone(), lin.weight.grad.clone()))
            lin.weight.grad = None
        return outs, lin

    a, _ = run(R.CustomRecipe(qfactory=both))
    b, _ = run(R.DelayedScaling(amax_history_len=4, margin=0))
    for ta, tb in zip(a, b):
        for u, v in zip(ta, tb):
            torch.testing.assert_close(u, v, rtol=0, atol=0)
    c, lin = run(R.CustomRecipe(qfactory=mixed))
    for (yc, gx, gw), (yb, _, _) in zip(c, b):
        assert torch.isfinite(gx).all() and torch.isfinite(gw).all()
        assert (yc - yb).abs().max() < 0.1 * yb.abs().max()
    inner = lin._states["scaling_fwd"].delayed
    assert inner is not None and inner.amax_history.shape[1] == 2       # input and weight: one row-wise child each
    assert float(inner.scale.min()) > 0 and not torch.equal(inner.scale, torch.ones_like(inner.scale))
    with pytest.raises(RuntimeError, match="unresolved"):
        te.HybridQuantizer(rowwise_quantizer=req, columnwise_quantizer=MXFP8Quantizer())(torch.randn(32, 32))
