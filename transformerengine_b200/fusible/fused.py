"""Fused implementations that ``Sequential`` substitutes for runs of basic operations, forward AND
backward (reference: ``pytorch/ops/fused/forward_linear_bias_activation.py``,
``forward_linear_bias_add.py``, ``forward_linear_scale_add.py``, ``backward_activation_bias.py``,
``backward_linear_add.py``, ``backward_linear_scale.py``, ``backward_add_rmsnorm.py``).

``LinearChain`` covers ``Linear (+ Bias) (+ ConstantScale) (+ Activation) (+ AddExtraInput)``:

* forward: one GEMM whose epilogue applies the scale (``alpha``) and the bias, then the activation
  kernel, then the residual add;
* backward: ONE kernel computes the activation gradient, the bias gradient (column sums) and the
  quantized copies that the dgrad / wgrad GEMMs read (``activation_bwd(..., want_dbias=True,
  quantizer=...)``); the scale is folded into the GEMMs' ``alpha``; the residual branch receives the
  incoming gradient untouched.

``ForkNorm`` covers ``MakeExtraOutput, RMSNorm / LayerNorm``: the norm backward kernel adds the
gradient of the forked branch while it writes dx (no separate add pass).

``GroupedMLP`` covers ``GroupedLinear, ScaledSwiGLU, GroupedLinear`` (an MoE expert MLP, reference
``pytorch/ops/fused/grouped_mlp.py``): the split sizes are read once for both grouped GEMMs and the scaled
activation is one kernel forward and one kernel for the input gradient.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops as K
from ..modules import _functional as F
from ..quantization import FP8GlobalStateManager


class _LinearChainFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, extra, module, wq, scale, act):  # type: ignore[override]
        cfg = module.cfg
        adt = cfg.activation_dtype
        lead = x.shape[:-1]
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.dtype != adt:
            x2d = x2d.to(adt)
        grad_on = any(ctx.needs_input_grad)
        need_wgrad = weight.requires_grad and grad_on
        in_q = module.get_quantizer(True, 0)
        xq = F.quantize_for_gemm(x2d, in_q, True, need_wgrad)
        a, b = F.as_operand(xq, "rowwise"), F.as_operand(wq, "rowwise")
        pre = K.gemm_nt(a, b, out_dtype=adt, bias=bias, alpha=scale)      # alpha and bias in the GEMM epilogue
        y = pre
        if act is not None:
            y, _ = K.activation_fwd(pre, act)
            y = y.to(adt)
        if extra is not None:
            y = y + extra.reshape(y.shape).to(y.dtype)
        if grad_on:
            keep_x = xq if need_wgrad else None
            if F._is_q(keep_x) and keep_x.get_usages()["columnwise"]:
                keep_x.update_usage(rowwise_usage=False)
            from ..tensor.base import prepare_for_saving

            flat, objs = prepare_for_saving(keep_x)
            ctx.save_for_backward(*flat, weight, pre if act is not None else None)
            ctx.objs = objs
            ctx.wq = wq if F._is_q(wq) else None
            ctx.module, ctx.scale, ctx.act = module, scale, act
            ctx.has_bias, ctx.has_extra = bias is not None, extra is not None
            ctx.bias_dtype = bias.dtype if bias is not None else None
            ctx.x_shape, ctx.extra_shape = x.shape, (extra.shape if extra is not None else None)
            ctx.fp8 = module.fp8
            ctx.need_wgrad = need_wgrad
            ctx.need_dgrad = x.requires_grad
            ctx.reduce_bwd_amax = FP8GlobalStateManager.is_first_fp8_module() if module.fp8 else False
        return y.reshape(*lead, y.shape[-1])

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        from ..tensor.base import restore_from_saved

        saved = list(ctx.saved_tensors)
        pre = saved.pop()
        weight = saved.pop()
        (keep_x,) = restore_from_saved(ctx.objs, saved)
        module = ctx.module
        cfg = module.cfg
        adt = cfg.activation_dtype
        w_use = ctx.wq if ctx.wq is not None else weight
        dy2d = dy.reshape(-1, dy.shape[-1]).to(adt).contiguous()
        d_extra = dy.reshape(ctx.extra_shape) if ctx.has_extra else None   # residual branch: gradient passes through
        go_q = module.get_quantizer(False, 0) if ctx.fp8 else None
        db = None
        if ctx.act is not None:
            # activation gradient + bias gradient + quantized copies in one kernel
            if go_q is not None:
                go_q.set_usage(rowwise=ctx.need_dgrad, columnwise=ctx.need_wgrad)
                go_q.internal = True
            dpre_hp, dpre_q, db = K.activation_bwd(dy2d, pre, ctx.act, quantizer=go_q, want_hp=go_q is None,
                                                   want_dbias=ctx.has_bias)
            dpre = dpre_q if dpre_q is not None else dpre_hp
        else:
            if ctx.has_bias:
                db = F.bias_grad(dy2d, ctx.bias_dtype)
            dpre = F.quantize_for_gemm(dy2d, go_q, ctx.need_dgrad, ctx.need_wgrad)
        if db is not None:
            db = db.to(ctx.bias_dtype)
        dx = dw = None
        if ctx.need_dgrad:
            a, b = F.as_operand(dpre, "rowwise"), F.as_operand(w_use, "columnwise")
            dx = K.gemm_nt(a, b, out_dtype=adt, alpha=ctx.scale).reshape(ctx.x_shape)   # scale folded into dgrad
        if ctx.need_wgrad:
            a, b = F.as_operand(dpre, "columnwise"), F.as_operand(keep_x, "columnwise")
            dw = K.gemm_nt(a, b, out_dtype=weight.dtype if weight.dtype in (torch.bfloat16, torch.float16, torch.float32)
                           else adt, alpha=ctx.scale).reshape(weight.shape)
        if ctx.fp8 and ctx.reduce_bwd_amax:
            FP8GlobalStateManager.reduce_and_update_fp8_tensors(forward=False)
        return dx, dw, db, d_extra, None, None, None, None


class LinearChain(torch.nn.Module):
    """Stand-in for ``Linear (+Bias) (+ConstantScale) (+Activation) (+AddExtraInput)``; the parameters stay
    with the basic operations."""

    is_fused_op = True

    def __init__(self, linear, bias_op=None, scale: float = 1.0, act: Optional[str] = None, add_extra: bool = False):
        super().__init__()
        self._lin = [linear]
        self._bias_op = [bias_op]
        self.scale, self.act = float(scale), act
        self.num_extra_inputs = 1 if add_extra else 0
        self.num_extra_outputs = 0
        self.span = 1 + (bias_op is not None) + (scale != 1.0) + (act is not None) + add_extra
        self.fusion = "linear" + ("_bias" if (bias_op is not None or getattr(linear, "bias", None) is not None) else "") \
            + ("_scale" if scale != 1.0 else "") + (f"_{act}" if act else "") + ("_add" if add_extra else "")

    def forward(self, x, *extra):
        lin = self._lin[0]
        lin.prepare_forward(num_gemms=1)
        lin.cfg.activation_dtype = torch.get_autocast_gpu_dtype() if torch.is_autocast_enabled() else x.dtype
        weight, bias = lin._get_weight_bias()
        if self._bias_op[0] is not None:
            assert bias is None or not lin.apply_bias, "Linear with a bias followed by a Bias operation"
            bias = self._bias_op[0].bias
        elif not lin.apply_bias:
            bias = None
        wq = lin.get_quantized_weight(weight, lin.get_quantizer(True, 1), cache_name="weight")
        adt = lin.cfg.activation_dtype
        if isinstance(wq, torch.Tensor) and not F._is_q(wq) and wq.dtype != adt:
            wq = wq.to(adt)
        # the pattern matcher only combines a scale with a bias-free linear, so y = scale * (x W^T) (+ b if scale == 1)
        b_use = bias.to(adt) if bias is not None else None
        return _LinearChainFn.apply(x, weight, b_use, extra[0] if extra else None, lin, wq, self.scale, self.act)


class _ForkNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, zero_centered, layernorm):  # type: ignore[override]
        x2 = x.contiguous()
        y, _, mu, rs = K.norm_fwd(x2, gamma, beta, eps, zero_centered, layernorm)
        ctx.save_for_backward(x2, gamma, mu, rs)
        ctx.zc, ctx.ln = zero_centered, layernorm
        return y, x2.view_as(x2)  # (normalized, forked copy of the input)

    @staticmethod
    def backward(ctx, dy, dfork):  # type: ignore[override]
        x, gamma, mu, rs = ctx.saved_tensors
        # dx = norm_bwd(dy) + dfork in the norm backward kernel
        dx, dg, db = K.norm_bwd(dy.contiguous(), x, mu, rs, gamma, ctx.zc, ctx.ln,
                                add=dfork.contiguous() if dfork is not None else None)
        return dx, dg, db, None, None, None


class ForkNorm(torch.nn.Module):
    """Stand-in for ``MakeExtraOutput, RMSNorm/LayerNorm``: returns (normalized, input) and fuses the add
    of the two incoming gradients into the norm backward."""

    is_fused_op = True

    def __init__(self, norm, layernorm: bool):
        super().__init__()
        self._norm = [norm]
        self.layernorm = layernorm
        self.span, self.num_extra_inputs, self.num_extra_outputs, self.fusion = 2, 0, 1, "fork_norm"

    def forward(self, x):
        n = self._norm[0]
        w, b = n.weight, n.bias
        if w.dtype != x.dtype and w.dtype != torch.float32:
            w = w.to(x.dtype)
            b = b.to(x.dtype) if b is not None else None
        return _ForkNormFn.apply(x, w, b, n.eps, n.zero_centered_gamma, self.layernorm)


class GroupedMLP(torch.nn.Module):
    """Stand-in for ``GroupedLinear, ScaledSwiGLU, GroupedLinear``: ``forward(x, split_sizes, scales, split_sizes)``
    (the extra inputs of the three basic operations, in order).  The parameters stay with the basic operations."""

    is_fused_op = True

    def __init__(self, fc1, act, fc2):
        super().__init__()
        self._ops = [fc1, act, fc2]
        self.span, self.num_extra_inputs, self.num_extra_outputs, self.fusion = 3, 3, 0, "grouped_mlp"

    def forward(self, x, splits1, scales, splits2):
        from .ops import _ScaledGluFn, _splits_list

        fc1, act, fc2 = self._ops
        m_splits = _splits_list(splits1)                      # one host read for both grouped GEMMs
        if splits2 is not splits1:
            assert _splits_list(splits2) == m_splits, "both grouped linears of an expert MLP see the same slabs"
        h = fc1.impl(x, m_splits)
        h = _ScaledGluFn.apply(h, scales.reshape(-1), act.act_name)
        return fc2.impl(h, m_splits)
