"""``LayerNorm`` / ``RMSNorm`` modules and ``LayerNormLinear`` (norm fused in front of a
linear layer; the normalised activations go straight to the quantized format the
GEMM reads).  Reference API: ``pytorch/module/layernorm_linear.py:1207``,
``layernorm.py``, ``rmsnorm.py``."""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple, Union

import torch

from .. import ops
from ..parallel import distributed as D
from ..quantization import FP8GlobalStateManager
from ..tensor.base import QuantizedTensorStorage, prepare_for_saving, restore_from_saved
from . import _functional as F
from .base import TransformerEngineBaseModule, WeightGradStore, get_default_init_method
from .linear import _ConcatView


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, zero_centered, layernorm):  # type: ignore[override]
        y, _, mu, rs = ops.norm_fwd(x, gamma, beta, eps, zero_centered, layernorm)
        ctx.save_for_backward(x, gamma, mu, rs)
        ctx.zc, ctx.ln = zero_centered, layernorm
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, gamma, mu, rs = ctx.saved_tensors
        dx, dg, db = ops.norm_bwd(dy.contiguous(), x, mu, rs, gamma, ctx.zc, ctx.ln)
        return dx, dg, db, None, None, None


class _NormBase(torch.nn.Module):
    _layernorm = False

    def __init__(self, normalized_shape=None, eps: float = 1e-5, sequence_parallel: bool = False,
                 params_dtype: Optional[torch.dtype] = None, zero_centered_gamma: bool = False,
                 device: Union[torch.device, str] = None, hidden_size: Optional[int] = None, **kwargs):
        super().__init__()
        if normalized_shape is None:
            normalized_shape = hidden_size
        if isinstance(normalized_shape, (tuple, list)):
            assert len(normalized_shape) == 1
            normalized_shape = normalized_shape[0]
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.eps, self.zero_centered_gamma = eps, zero_centered_gamma
        self.sequence_parallel = sequence_parallel
        init = torch.zeros if zero_centered_gamma else torch.ones
        self.weight = torch.nn.Parameter(init(normalized_shape, device=device, dtype=params_dtype))
        if self._layernorm:
            self.bias = torch.nn.Parameter(torch.zeros(normalized_shape, device=device, dtype=params_dtype))
        else:
            self.register_parameter("bias", None)
        for p in (self.weight, self.bias):
            if p is not None:
                setattr(p, "sequence_parallel", sequence_parallel)

    def reset_parameters(self, defer_init: bool = False) -> None:
        """Norm weights to their identity value (0 with ``zero_centered_gamma``), bias to 0; parameters created on
        the ``meta`` device are materialised first."""
        if defer_init:
            return
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        for name in ("weight", "bias"):
            p = getattr(self, name)
            if p is not None and p.device.type == "meta":
                new = torch.nn.Parameter(torch.empty(tuple(p.shape), dtype=p.dtype, device=dev))
                setattr(new, "sequence_parallel", getattr(p, "sequence_parallel", False))
                self.register_parameter(name, new)
        with torch.no_grad():
            self.weight.fill_(0.0 if self.zero_centered_gamma else 1.0)
            if self.bias is not None:
                self.bias.zero_()

    def forward(self, inp: torch.Tensor) -> torch.Tensor:
        w, b = self.weight, self.bias
        if w.dtype != inp.dtype and w.dtype != torch.float32:
            w = w.to(inp.dtype)
            b = b.to(inp.dtype) if b is not None else None
        return _NormFn.apply(inp, w, b, self.eps, self.zero_centered_gamma, self._layernorm)


class LayerNorm(_NormBase):
    """y = (x - E[x]) / sqrt(Var[x] + eps) * gamma + beta over the last dim."""

    _layernorm = True


class RMSNorm(_NormBase):
    """y = x / sqrt(mean(x^2) + eps) * gamma over the last dim."""

    _layernorm = False


class _LayerNormLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, ln_w, ln_b, weight, bias, module, cfg, wq, return_ln_out, is_first_microbatch):  # type: ignore[override]
        hidden = inp.shape[-1]
        x2d = inp.reshape(-1, hidden)
        if x2d.dtype != cfg.activation_dtype:
            x2d = x2d.to(cfg.activation_dtype)
        x2d = x2d.contiguous()
        fp8 = module.fp8
        in_q = module.get_quantizer(True, 0)
        grad_on = any(ctx.needs_input_grad)
        need_wgrad = weight.requires_grad and grad_on
        sp_gather = cfg.parallel_mode == "column" and cfg.sequence_parallel and cfg.tp_size > 1
        # recipe.backward_override: quantized forward, unquantized backward GEMMs on the original ("high_precision")
        # or on the dequantized forward operands ("dequantized")
        override = module.backward_override() if (fp8 and grad_on) else None
        # sequence parallel with fused collectives and MXFP8: the norm writes this rank's rows quantized
        # (both copies in one pass), the all-gather moves FP8 and the columnwise copy is kept for wgrad
        # (with a backward override the backward needs no quantized copy: plain gather of the quantized rows)
        sp_fused_q = sp_gather and isinstance(in_q, F.MXFP8Quantizer) and F._fused_comm_ok(cfg, x2d.shape[0], x2d) \
            and x2d.shape[0] % 128 == 0 and override is None
        if in_q is not None:
            in_q.set_usage(rowwise=True, columnwise=need_wgrad and (not sp_gather or sp_fused_q) and override is None)
            in_q.internal = True
        ln_hp, ln_q, mu, rs = ops.norm_fwd(x2d, ln_w, ln_b, module.eps, module.zero_centered_gamma,
                                           module.normalization == "LayerNorm",
                                           quantizer=in_q if (not sp_gather or sp_fused_q) else None,
                                           want_hp=return_ln_out or in_q is None or (sp_gather and not sp_fused_q)
                                           or override == "high_precision")
        out = None
        ln_total = None
        ln_local = ln_q if (sp_fused_q and ln_q is not None) else ln_hp
        if sp_gather:
            if override is None and F._fused_comm_ok(cfg, x2d.shape[0], x2d):
                res = F.fused_all_gather_gemm(ln_local, F.as_operand(wq, "rowwise"), bias, cfg, in_q,
                                              cfg.activation_dtype, "fprop", columnwise=need_wgrad)
                if res is not None:
                    out, ln_local = res[0], res[1]
            if out is None:
                ln_total = F.gather_input(ln_local, cfg, in_q, True, need_wgrad and override is None)
        else:
            ln_total = ln_q if ln_q is not None else ln_hp
        if out is None:
            out, _ = F.linear_fprop(ln_total, wq, bias, cfg, cfg.activation_dtype)
        if grad_on:
            keep = (ln_local if sp_gather else ln_total) if need_wgrad else None
            if override == "high_precision" and need_wgrad:
                keep = ln_hp
            elif override == "dequantized" and need_wgrad and sp_gather:
                keep = F.quantize_for_gemm(ln_hp, in_q, True, False)    # this rank's rows as the forward saw them
            if F._is_q(keep) and keep.get_usages()["columnwise"]:
                keep.update_usage(rowwise_usage=False)
            ctx.wq = wq if F._is_q(wq) else None  # cached object shared across calls: not stripped
            flat, objs = prepare_for_saving(keep)
            ctx.save_for_backward(*flat, x2d, ln_w, ln_b, mu, rs, weight, bias)
            ctx.objs = objs
            ctx.module, ctx.cfg, ctx.fp8 = module, cfg, fp8 and override is None
            ctx.override = override
            ctx.inp_shape = inp.shape
            ctx.sp_gather = sp_gather
            ctx.requires_wgrad = need_wgrad
            ctx.return_ln_out = return_ln_out
            ctx.reduce_bwd_amax = FP8GlobalStateManager.is_first_fp8_module() if fp8 else False
        lead = inp.shape[:-1]
        if sp_gather:
            lead = (lead[0] * cfg.tp_size,) + tuple(lead[1:])
        out = out.reshape(*lead, out.shape[-1])
        if return_ln_out:
            return out, ln_hp.reshape(inp.shape)
        return out

    @staticmethod
    def backward(ctx, grad_output, *extra):  # type: ignore[override]
        saved = list(ctx.saved_tensors)
        bias = saved.pop(); weight = saved.pop(); rs = saved.pop(); mu = saved.pop()
        ln_b = saved.pop(); ln_w = saved.pop(); x2d = saved.pop()
        (keep,) = restore_from_saved(ctx.objs, saved)
        wq = ctx.wq
        module, cfg = ctx.module, ctx.cfg
        w_use = wq if wq is not None else weight
        if ctx.override is not None:
            adt = cfg.activation_dtype
            hp = lambda t: t.dequantize(dtype=adt) if F._is_q(t) else (t if t.dtype == adt else t.to(adt))  # noqa: E731
            w_use = hp(weight) if ctx.override == "high_precision" else hp(w_use)
            keep = hp(keep) if keep is not None else None
        dy2d = grad_output.reshape(-1, grad_output.shape[-1]).to(cfg.activation_dtype).contiguous()
        go_q = module.get_quantizer(False, 0) if ctx.fp8 else None
        db = F.bias_grad(dy2d, bias.dtype) if bias is not None else None
        dyq = F.quantize_for_gemm(dy2d, go_q, True, ctx.requires_wgrad)
        dln, h, x_total = F.linear_dgrad(dyq, w_use, cfg, cfg.activation_dtype, async_comm=True,
                                         side=keep if (ctx.sp_gather and ctx.requires_wgrad) else None)
        dw = None
        if ctx.requires_wgrad:
            xw = keep
            if ctx.sp_gather:
                in_q = module.get_quantizer(True, 0) if ctx.fp8 else None
                xw = F.gathered_wgrad_input(keep, x_total, cfg, in_q)
            dw = F.linear_wgrad(dyq, xw, weight, cfg)
        if h is not None:
            h.wait()
        if ctx.return_ln_out and extra and extra[0] is not None:
            dln = dln + extra[0].reshape(dln.shape).to(dln.dtype)
        dx, dg, dbeta = ops.norm_bwd(dln, x2d, mu, rs, ln_w, module.zero_centered_gamma,
                                     module.normalization == "LayerNorm")
        if ctx.fp8 and ctx.reduce_bwd_amax:
            FP8GlobalStateManager.reduce_and_update_fp8_tensors(forward=False)
        return dx.reshape(ctx.inp_shape), dg, dbeta, dw, db, None, None, None, None, None


class LayerNormLinear(TransformerEngineBaseModule):
    """LayerNorm/RMSNorm followed by a linear layer.  Parameters: ``layer_norm_weight``,
    ``layer_norm_bias``, ``weight``, ``bias`` (or ``{name}_weight`` with ``parameters_split``)."""

    def __init__(self, in_features: int, out_features: int, eps: float = 1e-5, sequence_parallel: bool = False,
                 fuse_wgrad_accumulation: bool = False, tp_group=None, tp_size: int = 1,
                 get_rng_state_tracker: Optional[Callable] = None, init_method: Optional[Callable] = None,
                 bias: bool = True, normalization: str = "LayerNorm", return_bias: bool = False,
                 params_dtype: Optional[torch.dtype] = None, parallel_mode: Optional[str] = None,
                 return_layernorm_output: bool = False, return_layernorm_output_gathered: bool = False,
                 parameters_split: Optional[Union[Tuple[str, ...], Dict[str, int]]] = None,
                 zero_centered_gamma: bool = False, device: Union[torch.device, str] = None,
                 ub_overlap_ag: bool = False, ub_overlap_rs_dgrad: bool = False, ub_bulk_wgrad: bool = False,
                 ub_bulk_dgrad: bool = False, ub_name: Optional[str] = None, delay_wgrad_compute: bool = False,
                 symmetric_ar_type: Optional[str] = None, name: Optional[str] = None,
                 ub_overlap_rs: bool = False) -> None:
        super().__init__()
        # with sequence parallelism the returned normalized output is this rank's rows, or all rows (gathered over
        # the tensor-parallel group; gradients reduce-scatter back) with return_layernorm_output_gathered
        self.return_layernorm_output_gathered = return_layernorm_output_gathered
        if symmetric_ar_type is not None:
            raise NotImplementedError("symmetric_ar_type: use te.initialize_ub (fused GEMM + collective kernels) instead")
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        assert normalization in ("LayerNorm", "RMSNorm")
        self.in_features, self.out_features = in_features, out_features
        self.eps, self.normalization, self.zero_centered_gamma = eps, normalization, zero_centered_gamma
        self.use_bias, self.return_bias = bias, return_bias
        self.apply_bias = bias and not return_bias
        self.return_layernorm_output = return_layernorm_output
        self.fuse_wgrad_accumulation = fuse_wgrad_accumulation
        self.name = name
        if tp_group is None:
            self.tp_size = tp_size
            if tp_size == 1:
                self.set_tensor_parallel_group(tp_group)
        else:
            self.set_tensor_parallel_group(tp_group)
        assert parallel_mode in (None, "column", "row")
        self.parallel_mode = parallel_mode
        if parallel_mode == "column":
            self.out_features = out_features // self.tp_size
        elif parallel_mode == "row":
            self.in_features = in_features // self.tp_size
        self.sequence_parallel = (self.tp_size > 1) and sequence_parallel
        self.wgrad_store = WeightGradStore(delay_wgrad_compute)
        self.activation_dtype = params_dtype
        init_method = init_method or get_default_init_method()
        ln_init = torch.zeros if zero_centered_gamma else torch.ones
        self.layer_norm_weight = torch.nn.Parameter(ln_init(in_features, device=device, dtype=params_dtype))
        setattr(self.layer_norm_weight, "sequence_parallel", self.sequence_parallel)
        if normalization == "LayerNorm":
            self.layer_norm_bias = torch.nn.Parameter(torch.zeros(in_features, device=device, dtype=params_dtype))
            setattr(self.layer_norm_bias, "sequence_parallel", self.sequence_parallel)
        else:
            self.layer_norm_bias = None
        if parameters_split is None:
            names, sizes = ("",), (self.out_features,)
        elif isinstance(parameters_split, dict):
            names = tuple(f"{k}_" for k in parameters_split)
            sizes = tuple(parameters_split.values())
            if parallel_mode == "column":
                sizes = tuple(s // self.tp_size for s in sizes)
        else:
            names = tuple(f"{k}_" for k in parameters_split)
            sizes = (self.out_features // len(names),) * len(names)
        assert sum(sizes) == self.out_features
        self.weight_names = [f"{n}weight" for n in names]
        self.bias_names = [f"{n}bias" for n in names]
        self._split_sizes = sizes
        wt = torch.empty(self.out_features, self.in_features, device=device, dtype=params_dtype)
        bt = torch.zeros(self.out_features, device=device, dtype=params_dtype) if bias else None
        off = 0
        for n, s in zip(names, sizes):
            w = wt[off:off + s]
            if str(device) != "meta":
                if get_rng_state_tracker is not None and parallel_mode is not None:
                    with get_rng_state_tracker().fork():
                        init_method(w)
                else:
                    init_method(w)
            p = torch.nn.Parameter(w)
            if parallel_mode is not None:
                D.set_tensor_model_parallel_attributes(p, True, 0 if parallel_mode == "column" else 1, 1)
            self.register_parameter(f"{n}weight", p)
            if bias:
                bp = torch.nn.Parameter(bt[off:off + s])
                if parallel_mode == "column":
                    D.set_tensor_model_parallel_attributes(bp, True, 0, 1)
                self.register_parameter(f"{n}bias", bp)
            off += s
        self._fused_weight_storage = wt if len(names) > 1 else None

        def init_w(w, f=init_method):
            if get_rng_state_tracker is not None and parallel_mode is not None:
                with get_rng_state_tracker().fork():
                    return f(w)
            return f(w)

        self._init_fns = {"layer_norm_weight": torch.nn.init.zeros_ if zero_centered_gamma else torch.nn.init.ones_}
        if normalization == "LayerNorm":
            self._init_fns["layer_norm_bias"] = torch.nn.init.zeros_
        self._init_fns.update({n: init_w for n in self.weight_names})
        if bias:
            self._init_fns.update({n: torch.nn.init.zeros_ for n in self.bias_names})
        if self.primary_weights_in_fp8:
            self._quantize_primary_weights(self.weight_names)
            self._fused_weight_storage = None
        self.cfg = F.LinearConfig(parallel_mode=self.parallel_mode, sequence_parallel=self.sequence_parallel,
                                  tp_group=self.tp_group, tp_size=self.tp_size,
                                  fuse_wgrad_accumulation=fuse_wgrad_accumulation, activation_dtype=params_dtype,
                                  wgrad_store=self.wgrad_store, name=name or "")

    def set_tensor_parallel_group(self, tp_group) -> None:
        super().set_tensor_parallel_group(tp_group)
        if hasattr(self, "cfg"):
            self.cfg.tp_group, self.cfg.tp_size = self.tp_group, self.tp_size

    def _get_weight_bias(self):
        ws = [getattr(self, n) for n in self.weight_names]
        if len(ws) == 1:
            w = ws[0]
        elif self._fused_weight_storage is not None and all(
                x.data_ptr() == self._fused_weight_storage[sum(self._split_sizes[:i])].data_ptr()
                for i, x in enumerate(ws)):
            w = _ConcatView.apply(self._fused_weight_storage, *ws)
        else:
            w = torch.cat([x.dequantize() if isinstance(x, QuantizedTensorStorage) else x for x in ws], dim=0)
        b = None
        if self.use_bias:
            bs = [getattr(self, n) for n in self.bias_names]
            b = bs[0] if len(bs) == 1 else torch.cat(bs, dim=0)
        return w, b

    def forward(self, inp: torch.Tensor, is_first_microbatch: Optional[bool] = None, fp8_output: bool = False,
                fp8_grad: bool = False):
        if fp8_output or fp8_grad:
            raise NotImplementedError("fp8_output / fp8_grad: quantized layer outputs and input gradients are not "
                                      "implemented; the next layer quantizes its own input")
        self.prepare_forward(num_gemms=1)
        self.cfg.activation_dtype = torch.get_autocast_gpu_dtype() if torch.is_autocast_enabled() else inp.dtype
        weight, bias = self._get_weight_bias()
        wq = self.get_quantized_weight(weight, self.get_quantizer(True, 1), cache_name="weight",
                                       is_first_microbatch=is_first_microbatch)
        adt = self.cfg.activation_dtype
        if not isinstance(wq, QuantizedTensorStorage) and wq.dtype != adt:
            wq = wq.to(adt)
        b_use = bias.to(adt) if (self.apply_bias and bias is not None) else None
        ln_w, ln_b = self.layer_norm_weight, self.layer_norm_bias
        if ln_w.dtype not in (adt, torch.float32):
            ln_w = ln_w.to(adt)
            ln_b = ln_b.to(adt) if ln_b is not None else None
        res = _LayerNormLinear.apply(inp, ln_w, ln_b, weight, b_use, self, self.cfg, wq,
                                     self.return_layernorm_output, is_first_microbatch)
        out, ln_out = (res if self.return_layernorm_output else (res, None))
        if ln_out is not None and self.return_layernorm_output_gathered and self.sequence_parallel \
                and self.parallel_mode == "column":
            from ..parallel.distributed import gather_rows_with_grad
            ln_out = gather_rows_with_grad(ln_out, self.cfg.tp_group)
        if self.return_bias:
            if self.return_layernorm_output:
                return out, (bias.to(adt) if bias is not None else None), ln_out
            return out, (bias.to(adt) if bias is not None else None)
        if self.return_layernorm_output:
            return out, ln_out
        return out
