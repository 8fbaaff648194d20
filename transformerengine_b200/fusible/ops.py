"""Basic fusible operations (reference: ``pytorch/ops/basic/*.py``).

Every operation is an ``nn.Module`` with ``forward(x, *extra_inputs)``.  ``num_extra_inputs`` /
``num_extra_outputs`` tell ``Sequential`` how many additional tensors an operation consumes
from / adds to the call.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import ops as K
from ..modules.layernorm_linear import LayerNorm as _TELayerNorm
from ..modules.layernorm_linear import RMSNorm as _TERMSNorm
from ..modules.linear import Linear as _TELinear
from ..parallel import distributed as D


class FusibleOperation(torch.nn.Module):
    """Base class: an operation that ``Sequential`` may replace by a fused implementation."""

    num_extra_inputs = 0
    num_extra_outputs = 0

    @property
    def is_fused_op(self) -> bool:
        return False


class BasicLinear(_TELinear, FusibleOperation):
    """``y = x W^T`` (no bias); parameter ``weight``."""

    def __init__(self, in_features, out_features, *, device=None, dtype=None, tensor_parallel_mode=None,
                 tensor_parallel_group=None, sequence_parallel=False, accumulate_into_main_grad=False, **kw):
        super().__init__(in_features, out_features, bias=False, params_dtype=dtype, device=device,
                         parallel_mode=tensor_parallel_mode, tp_group=tensor_parallel_group,
                         sequence_parallel=sequence_parallel, fuse_wgrad_accumulation=accumulate_into_main_grad, **kw)


class Linear(_TELinear, FusibleOperation):
    """``y = x W^T + b``; parameters ``weight`` and ``bias``."""

    def __init__(self, in_features, out_features, *, bias=True, device=None, dtype=None, tensor_parallel_mode=None,
                 tensor_parallel_group=None, sequence_parallel=False, accumulate_into_main_grad=False, **kw):
        super().__init__(in_features, out_features, bias=bias, params_dtype=dtype, device=device,
                         parallel_mode=tensor_parallel_mode, tp_group=tensor_parallel_group,
                         sequence_parallel=sequence_parallel, fuse_wgrad_accumulation=accumulate_into_main_grad, **kw)


class Bias(FusibleOperation):
    def __init__(self, size, *, device=None, dtype=None):
        super().__init__()
        self.bias = torch.nn.Parameter(torch.zeros(size, device=device, dtype=dtype))

    def forward(self, x):
        return x + self.bias.to(x.dtype)


class LayerNorm(_TELayerNorm, FusibleOperation):
    def __init__(self, normalized_shape, *, eps=1e-5, device=None, dtype=None, zero_centered_gamma=False, **kw):
        n = normalized_shape if isinstance(normalized_shape, int) else normalized_shape[-1]
        super().__init__(n, eps=eps, params_dtype=dtype, device=device, zero_centered_gamma=zero_centered_gamma, **kw)


class RMSNorm(_TERMSNorm, FusibleOperation):
    def __init__(self, normalized_shape, *, eps=1e-5, device=None, dtype=None, zero_centered_gamma=False, **kw):
        n = normalized_shape if isinstance(normalized_shape, int) else normalized_shape[-1]
        super().__init__(n, eps=eps, params_dtype=dtype, device=device, zero_centered_gamma=zero_centered_gamma, **kw)


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name):  # type: ignore[override]
        y, _ = K.activation_fwd(x.contiguous(), name)
        ctx.save_for_backward(x)
        ctx.name = name
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        (x,) = ctx.saved_tensors
        dx, _, _ = K.activation_bwd(dy.contiguous(), x.contiguous(), ctx.name)
        return dx.to(x.dtype), None


class _Activation(FusibleOperation):
    act_name = "gelu"

    def __init__(self, *, cache_quantized_input: bool = False, glu_interleave_size: Optional[int] = None):
        super().__init__()
        self.cache_quantized_input = cache_quantized_input
        if glu_interleave_size is not None and not self.act_name.endswith("glu"):
            raise ValueError(f"glu_interleave_size is an option of the gated units, not of {type(self).__name__}")
        self.glu_interleave_size = glu_interleave_size      # block-interleaved gates / linear units: _deinterleave

    def forward(self, x):
        return _ActFn.apply(_deinterleave(x, self.glu_interleave_size), self.act_name)


class GELU(_Activation):
    act_name = "gelu"


class ReLU(_Activation):
    act_name = "relu"


class SiLU(_Activation):
    act_name = "silu"


class QGELU(_Activation):
    act_name = "qgelu"


class SReLU(_Activation):
    act_name = "srelu"


class SwiGLU(_Activation):
    act_name = "swiglu"


class GEGLU(_Activation):
    act_name = "geglu"


class ReGLU(_Activation):
    act_name = "reglu"


class QGEGLU(_Activation):
    act_name = "qgeglu"


class SReGLU(_Activation):
    act_name = "sreglu"


def _deinterleave(x, block: Optional[int]):
    """Block-interleaved gated input -> ``[gates | linear units]``: with ``glu_interleave_size = block`` the last
    dimension holds alternating blocks of ``block`` gate inputs and ``block`` linear inputs (``a1 a2 b1 b2 a3 a4 b3
    b4`` for block 2) instead of all gates followed by all linear units.  Plain reshapes, so autograd routes the
    gradient back into the interleaved layout.  (Reference: ``pytorch/ops/basic/swiglu.py:130-139``.)"""
    if block is None:
        return x
    n = x.shape[-1]
    if block <= 0 or n % (2 * block):
        raise ValueError(f"glu_interleave_size={block} does not divide the gated width {n} into gate / linear pairs")
    return x.reshape(-1, n // (2 * block), 2, block).transpose(1, 2).reshape(x.shape)


def _halves(x):
    """(gate input a, linear input b): the gating function applies to the FIRST half of the last dimension."""
    return x.float().chunk(2, dim=-1)


class _ElementwiseGLU(FusibleOperation):
    """Gated units outside the fused activation kernels' set: fp32 tensor math that autograd differentiates
    (a handful of element-wise launches on a GPU; the kernels cover gelu / silu / relu / qgelu / srelu gates)."""

    def __init__(self, *, cache_quantized_input: bool = False, glu_interleave_size: Optional[int] = None):
        super().__init__()
        self.glu_interleave_size = glu_interleave_size
        self.cache_quantized_input = cache_quantized_input

    def _glu(self, a, b):
        raise NotImplementedError

    def forward(self, x):
        a, b = _halves(_deinterleave(x, self.glu_interleave_size))
        return self._glu(a, b).to(x.dtype)


class GLU(_ElementwiseGLU):
    """``sigmoid(a) * b`` (reference: ``pytorch/ops/basic/activation.py``, ``GLU``)."""

    def _glu(self, a, b):
        return torch.sigmoid(a) * b


class ClampedSwiGLU(_ElementwiseGLU):
    """The GPT-OSS gated unit: ``a' = min(a, limit)``, ``b' = clamp(b, -limit, limit) + glu_linear_offset``,
    ``y = a' * sigmoid(alpha * a') * b'`` (reference: ``pytorch/ops/basic/swiglu.py``, ``ClampedSwiGLU``)."""

    def __init__(self, *, limit: float = 7.0, alpha: float = 1.702, glu_linear_offset: float = 1.0, **kw):
        super().__init__(**kw)
        self.limit, self.alpha, self.glu_linear_offset = float(limit), float(alpha), float(glu_linear_offset)

    def _glu(self, a, b):
        a = torch.clamp(a, max=self.limit)
        b = torch.clamp(b, -self.limit, self.limit) + self.glu_linear_offset
        return a * torch.sigmoid(self.alpha * a) * b


class SiTUGLU(_ElementwiseGLU):
    """Soft-capped SiLU gated unit: ``beta1 * tanh(a / beta1) * sigmoid(a) * beta2 * tanh(b / beta2)``
    (reference: ``pytorch/ops/basic/swiglu.py``, ``SiTUGLU``)."""

    def __init__(self, *, beta1: float = 4.0, beta2: float = 25.0, **kw):
        super().__init__(**kw)
        self.beta1, self.beta2 = float(beta1), float(beta2)
        for name, v in (("beta1", self.beta1), ("beta2", self.beta2)):
            if not (v > 0.0 and v != float("inf")):
                raise ValueError(f"{name} must be finite and positive, got {v}")

    def _glu(self, a, b):
        return self.beta1 * torch.tanh(a / self.beta1) * torch.sigmoid(a) * (self.beta2 * torch.tanh(b / self.beta2))


class _QuantizeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, quantizer, keep):  # type: ignore[override]
        q = quantizer(x)
        return q if keep else q.dequantize().to(x.dtype)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return g, None, None


class Quantize(FusibleOperation):
    """Quantize the activation with the recipe of the surrounding ``autocast`` (identity outside it)."""

    def __init__(self, forward: bool = True, backward: bool = False):
        super().__init__()
        self.quantize_forward, self.quantize_backward = forward, backward

    def forward(self, x):
        from ..quantization import FP8GlobalStateManager, RecipeState

        if not self.quantize_forward or not FP8GlobalStateManager.is_fp8_enabled():
            return x
        state = RecipeState.create(FP8GlobalStateManager.get_fp8_recipe(), mode="forward", num_quantizers=1)
        quantizer = state.make_quantizers()[0]
        quantizer.set_usage(rowwise=True, columnwise=False)
        return _QuantizeFn.apply(x, quantizer, False)


class Identity(FusibleOperation):
    def forward(self, x):
        return x


class Reshape(FusibleOperation):
    def __init__(self, shape: Sequence[int]):
        super().__init__()
        self.shape = tuple(shape)

    def forward(self, x):
        return x.reshape(self.shape)


class ConstantScale(FusibleOperation):
    def __init__(self, scale: float):
        super().__init__()
        self.scale = scale

    def forward(self, x):
        return x * self.scale


class Dropout(FusibleOperation):
    def __init__(self, p: float):
        super().__init__()
        self.p = p

    def forward(self, x):
        return torch.nn.functional.dropout(x, self.p, self.training)


class L2Normalization(FusibleOperation):
    def __init__(self, eps: float = 1e-6):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.square().sum(-1, keepdim=True) + self.eps)).to(x.dtype)


class AddExtraInput(FusibleOperation):
    """``y = x + extra`` (residual connection); consumes one extra input of the call."""

    num_extra_inputs = 1

    def __init__(self, *, in_place: bool = False):
        super().__init__()
        self.in_place = in_place

    def forward(self, x, extra):
        return x + extra


class MakeExtraOutput(FusibleOperation):
    """Pass ``x`` on and also return it as an extra output of the call."""

    num_extra_outputs = 1

    def forward(self, x):
        return x, x


def _splits_list(split_sizes) -> list:
    """Row counts per group as host ints (the grouped GEMM front end sizes its launches on the host)."""
    if isinstance(split_sizes, torch.Tensor):
        return [int(v) for v in split_sizes.tolist()]
    return [int(v) for v in split_sizes]


class GroupedLinear(FusibleOperation):
    """``y_i = x_i W_i^T + b_i`` over ``num_groups`` consecutive row slabs of the input (MoE experts).  The slab
    sizes arrive as the extra input ``split_sizes`` (tensor or list of ``num_groups`` ints).  Parameters
    ``weight{i}`` / ``bias{i}``.  (Reference: ``pytorch/ops/basic/grouped_linear.py:135``.)"""

    num_extra_inputs = 1

    def __init__(self, num_groups: int, in_features: int, out_features: int, *, bias: bool = True, device=None,
                 dtype=None, accumulate_into_main_grad: bool = False, single_grouped_weight: bool = False,
                 single_grouped_bias: bool = False, delay_wgrad_compute: bool = False, scale_bias: bool = False):
        super().__init__()
        if scale_bias:
            raise NotImplementedError("GroupedLinear(scale_bias=True) is not implemented")
        from ..modules.grouped_linear import GroupedLinear as _TEGroupedLinear

        self.num_groups, self.in_features, self.out_features = num_groups, in_features, out_features
        # the module owns the (stacked) parameters: they appear as impl.weight{i} / impl.bias{i} in the state dict
        # and as weight{i} / bias{i} attributes of this operation
        self.impl = _TEGroupedLinear(num_groups, in_features, out_features, bias=bias, params_dtype=dtype, device=device,
                                     fuse_wgrad_accumulation=accumulate_into_main_grad,
                                     single_grouped_weight=single_grouped_weight,
                                     single_grouped_bias=single_grouped_bias, delay_wgrad_compute=delay_wgrad_compute)

    def __getattr__(self, name):
        if name != "impl" and (name.startswith("weight") or name.startswith("bias")) and "impl" in self._modules:
            return getattr(self._modules["impl"], name)
        return super().__getattr__(name)

    def forward(self, x, split_sizes):
        return self.impl(x, _splits_list(split_sizes))


class _ScaledGluFn(torch.autograd.Function):
    """Gated activation with every output row multiplied by its scale: one kernel forward, one kernel for the
    input gradient (both take the row scale as a prologue), a row dot product for the scale gradient."""

    @staticmethod
    def forward(ctx, x, scales, act):  # type: ignore[override]
        y, _ = K.activation_fwd(x, act, row_scale=scales)
        ctx.save_for_backward(x, scales)
        ctx.act = act
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, scales = ctx.saved_tensors
        dy = dy.contiguous()
        dx, _, _ = K.activation_bwd(dy, x, ctx.act, row_scale=scales)
        dscales = None
        if ctx.needs_input_grad[1]:
            unscaled, _ = K.activation_fwd(x, ctx.act)
            dscales = K.row_dot(dy.reshape(-1, dy.shape[-1]), unscaled.to(dy.dtype).reshape(-1, dy.shape[-1])).to(scales.dtype).reshape(scales.shape)
        return dx.to(x.dtype), dscales, None


class ScaledSwiGLU(FusibleOperation):
    """``y = swiglu(x) * scales[:, None]``: the middle operation of an MoE expert MLP, where ``scales`` (extra
    input, one value per row) are the routing probabilities.  (Reference: ``pytorch/ops/basic/swiglu.py:598``.)"""

    num_extra_inputs = 1
    act_name = "swiglu"

    def __init__(self, glu_interleave_size: Optional[int] = None):
        super().__init__()
        self.glu_interleave_size = glu_interleave_size

    def forward(self, x, scales):
        return _ScaledGluFn.apply(_deinterleave(x, self.glu_interleave_size), scales.reshape(-1), self.act_name)


class _ScaledElementwise(FusibleOperation):
    """``y = f(x) * scales[..., None]`` with one extra input (a scale per row: the routing probability of an MoE
    expert MLP); fp32 tensor math that autograd differentiates, scale gradient included."""

    num_extra_inputs = 1

    def __init__(self, glu_interleave_size: Optional[int] = None, *, activation_recompute_in_mlp: bool = False):
        super().__init__()
        self.glu_interleave_size = glu_interleave_size
        if activation_recompute_in_mlp:
            raise NotImplementedError("activation_recompute_in_mlp: wrap the MLP in te.checkpoint instead")

    def _f(self, x):
        raise NotImplementedError

    def forward(self, x, scales):
        gated = type(self) is not ScaledSReLU      # the squared ReLU has no gate / linear halves to reorder
        y = self._f(_deinterleave(x, self.glu_interleave_size if gated else None).float())
        return (y * scales.float().reshape(*y.shape[:-1], 1)).to(x.dtype)


class ScaledSReLU(_ScaledElementwise):
    """Squared ReLU times a per-row scale (reference: ``pytorch/ops/basic/activation.py``, ``ScaledSReLU``)."""

    def _f(self, x):
        return torch.relu(x).square()


class ScaledClampedQGeGLU(_ScaledElementwise):
    """``ClampedSwiGLU`` numerics times a per-row scale (reference: ``pytorch/ops/basic/swiglu.py``)."""

    def __init__(self, glu_interleave_size: Optional[int] = None, *, limit: float = 7.0, alpha: float = 1.702,
                 glu_linear_offset: float = 1.0, **kw):
        super().__init__(glu_interleave_size, **kw)
        self._inner = ClampedSwiGLU(limit=limit, alpha=alpha, glu_linear_offset=glu_linear_offset)

    def _f(self, x):
        return self._inner._glu(*x.chunk(2, dim=-1))


class ScaledSiTUGLU(_ScaledElementwise):
    """``SiTUGLU`` times a per-row scale (reference: ``pytorch/ops/basic/swiglu.py``)."""

    def __init__(self, glu_interleave_size: Optional[int] = None, *, beta1: float = 4.0, beta2: float = 25.0, **kw):
        super().__init__(glu_interleave_size, **kw)
        self._inner = SiTUGLU(beta1=beta1, beta2=beta2)

    def _f(self, x):
        return self._inner._glu(*x.chunk(2, dim=-1))


class _CollFn(torch.autograd.Function):
    """Collective on dim 0 whose backward is the adjoint collective."""

    _ADJOINT = {"all_reduce": "identity", "all_gather": "reduce_scatter", "reduce_scatter": "all_gather"}

    @staticmethod
    def _run(kind, x, group):
        x = x.contiguous()
        n = dist.get_world_size(group)
        if kind == "identity":
            return x
        if kind == "all_reduce":
            y = x.clone()
            dist.all_reduce(y, group=group)
            return y
        if kind == "all_gather":
            y = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(y.view(-1), x.view(-1), group=group)
            return y
        y = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(y.view(-1), x.view(-1), group=group)
        return y

    @staticmethod
    def forward(ctx, x, kind, group):  # type: ignore[override]
        ctx.kind, ctx.group = kind, group
        return _CollFn._run(kind, x, group)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return _CollFn._run(_CollFn._ADJOINT[ctx.kind], g, ctx.group), None, None


class _Collective(FusibleOperation):
    kind = "all_reduce"

    def __init__(self, process_group=None):
        super().__init__()
        self.group = process_group

    def forward(self, x):
        if D.get_world_size(self.group) <= 1:
            return x
        return _CollFn.apply(x, self.kind, self.group)


class AllReduce(_Collective):
    kind = "all_reduce"


class AllGather(_Collective):
    kind = "all_gather"


class ReduceScatter(_Collective):
    kind = "reduce_scatter"
