"""``Linear``: y = x W^T + b with optional quantized GEMMs and tensor parallelism
(reference API: ``pytorch/module/linear.py:1474-1899``)."""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Dict, Optional, Tuple, Union

import torch

from .. import distributed_weight as DW
from ..parallel import distributed as D
from ..quantization import FP8GlobalStateManager
from ..tensor.base import QuantizedTensorStorage, prepare_for_saving, restore_from_saved
from . import _functional as F
from .base import TransformerEngineBaseModule, WeightGradStore, get_default_init_method, get_distributed_world_size


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, weight, bias, module, cfg: F.LinearConfig, is_first_microbatch, fp8_output, weight_q):  # type: ignore[override]
        dist_w = DW.is_distributed_weight(weight)   # the parameter is a shard; weight_q holds the full matrix
        in_features = (weight_q.size(-1) if F._is_q(weight_q) else weight_q.shape[-1]) if dist_w else weight.shape[-1]
        lead = inp.shape[:-1]
        x2d = inp.reshape(-1, in_features)
        fp8 = module.fp8
        in_q = module.get_quantizer(True, 0)
        grad_on = any(ctx.needs_input_grad)
        need_wgrad = weight.requires_grad and grad_on
        # recipe.backward_override: quantized forward, unquantized backward GEMMs on the original operands
        # ("high_precision") or on the dequantized forward operands ("dequantized")
        override = module.backward_override() if (fp8 and grad_on) else None
        if override is not None and dist_w:
            raise NotImplementedError("recipe.backward_override is not implemented for distributed weights")
        if x2d.dtype != cfg.activation_dtype and not F._is_q(x2d):
            x2d = x2d.to(cfg.activation_dtype)
        out = None
        sp_col = cfg.parallel_mode == "column" and cfg.sequence_parallel and cfg.tp_size > 1
        if sp_col:
            save_x = x2d  # local rows; gathered again in backward for wgrad
            if override is not None:
                # the backward runs on 16-bit operands: gather the quantized rows for this GEMM only and keep this
                # rank's rows unquantized ("high_precision") or as what the forward quantizer made of them
                xq = F.gather_input(x2d, cfg, in_q, True, False)
                if override == "dequantized" and need_wgrad:
                    save_x = F.quantize_for_gemm(x2d, in_q, True, False)
            elif F._fused_comm_ok(cfg, x2d.shape[0], x2d):
                res = F.fused_all_gather_gemm(x2d, F.as_operand(weight_q, "rowwise"), bias, cfg, in_q,
                                              cfg.activation_dtype, "fprop", columnwise=need_wgrad)
                if res is not None:
                    out, save_x = res[0], res[1]  # the quantized local rows carry the wgrad (columnwise) copy
            if out is None and override is None:
                xq = F.gather_input(x2d, cfg, in_q, True, need_wgrad)
        else:
            keep_original = (getattr(module, "save_original_input", False) or override == "high_precision") \
                and need_wgrad
            xq = F.quantize_for_gemm(x2d, in_q, True, need_wgrad and not keep_original and override is None)
            # save_original_input: keep the unquantized input and quantize its wgrad copy in the backward
            save_x = x2d if keep_original else xq
        if out is None:
            out, _ = F.linear_fprop(xq, weight_q, bias, cfg, cfg.activation_dtype)
        if grad_on:
            if F._is_q(save_x) and need_wgrad and override is None:
                save_x.update_usage(rowwise_usage=False) if save_x.get_usages()["columnwise"] else None
            keep_x = save_x if need_wgrad else None
            # the quantized weight is a cached object shared across calls: keep a reference, do not strip it
            ctx.wq = weight_q if (F._is_q(weight_q) and not dist_w) else None
            ctx.dist_w = dist_w
            flat, objs = prepare_for_saving(keep_x)
            ctx.save_for_backward(*flat, weight, bias)
            ctx.objs = objs
            ctx.module, ctx.cfg = module, cfg
            ctx.fp8 = fp8 and override is None
            ctx.override = override
            ctx.inp_shape = inp.shape
            ctx.use_bias = bias is not None
            ctx.requires_dgrad = inp.requires_grad
            ctx.requires_wgrad = need_wgrad
            ctx.gathered_in_fwd = sp_col
            ctx.reduce_bwd_amax = FP8GlobalStateManager.is_first_fp8_module() if fp8 else False
        out_lead = lead
        if cfg.parallel_mode == "row" and cfg.sequence_parallel and cfg.tp_size > 1:
            out_lead = (out.shape[0],)
            if len(lead) > 1:
                out_lead = (lead[0] // cfg.tp_size,) + tuple(lead[1:])
        elif cfg.parallel_mode == "column" and cfg.sequence_parallel and cfg.tp_size > 1:
            out_lead = (lead[0] * cfg.tp_size,) + tuple(lead[1:])
        return out.reshape(*out_lead, out.shape[-1])

    @staticmethod
    def backward(ctx, grad_output):  # type: ignore[override]
        saved = list(ctx.saved_tensors)
        bias = saved.pop()
        weight = saved.pop()
        (keep_x,) = restore_from_saved(ctx.objs, saved)
        wq = ctx.wq
        module, cfg = ctx.module, ctx.cfg
        w_use = wq if wq is not None else weight
        if ctx.override is not None:
            adt = cfg.activation_dtype
            hp = lambda t: t.dequantize(dtype=adt) if F._is_q(t) else (t if t.dtype == adt else t.to(adt))  # noqa: E731
            w_use = hp(weight) if ctx.override == "high_precision" else hp(w_use)
            keep_x = hp(keep_x) if keep_x is not None else None
        w_full = None
        if ctx.dist_w:  # assemble the full weight again instead of keeping it alive since the forward
            w_full = DW.materialize_weight_for_backward(weight)[0].detach()
            w_use = module.quantize_full_weight(w_full, cfg.activation_dtype)
        dy2d = grad_output.reshape(-1, grad_output.shape[-1])
        if dy2d.dtype != cfg.activation_dtype:
            dy2d = dy2d.to(cfg.activation_dtype)
        dy2d = dy2d.contiguous()
        go_q = module.get_quantizer(False, 0) if ctx.fp8 else None
        db = F.bias_grad(dy2d if not (cfg.parallel_mode == "row" and cfg.sequence_parallel and cfg.tp_size > 1)
                         else dy2d, bias.dtype) if ctx.use_bias else None
        dx = dw = None
        h = None
        if cfg.parallel_mode == "row" and cfg.sequence_parallel and cfg.tp_size > 1:
            if ctx.use_bias:
                db = F.bias_grad(dy2d, bias.dtype)
            dyq, dx = F.row_parallel_grad_output(dy2d, w_use, cfg, go_q, ctx.requires_dgrad, ctx.requires_wgrad,
                                                 cfg.activation_dtype)
        else:
            dyq = F.quantize_for_gemm(dy2d, go_q, ctx.requires_dgrad, ctx.requires_wgrad)
        x_total = None
        if ctx.requires_dgrad and dx is None:
            dx, h, x_total = F.linear_dgrad(dyq, w_use, cfg, cfg.activation_dtype, async_comm=True,
                                            side=keep_x if (ctx.gathered_in_fwd and ctx.requires_wgrad) else None)
        if ctx.requires_wgrad:
            xw = keep_x
            if ctx.gathered_in_fwd:
                in_q = module.get_quantizer(True, 0) if ctx.fp8 else None
                xw = F.gathered_wgrad_input(keep_x, x_total, cfg, in_q)
            elif ctx.fp8 and not F._is_q(keep_x) and getattr(module, "save_original_input", False):
                xw = F.quantize_for_gemm(keep_x, module.get_quantizer(True, 0), False, True)
            if ctx.dist_w:
                full_grad = F.linear_wgrad(dyq, xw, w_full, cfg)
                dw = DW.finalize_weight_grads(weight, [full_grad])[0]
            else:
                dw = F.linear_wgrad(dyq, xw, weight, cfg)
        if h is not None:
            h.wait()
        if dx is not None:
            dx = dx.reshape(ctx.inp_shape)
        if ctx.fp8 and ctx.reduce_bwd_amax:
            FP8GlobalStateManager.reduce_and_update_fp8_tensors(forward=False)
        return dx, dw, db, None, None, None, None, None


class Linear(TransformerEngineBaseModule):
    """Applies ``y = x A^T + b``.

    ``parallel_mode="column"`` shards ``out_features`` over ``tp_group``,
    ``"row"`` shards ``in_features``; with ``sequence_parallel`` the activations
    outside the GEMM are sharded along their first (sequence) dim.
    ``parameters_split`` exposes slices of the weight as separately named
    parameters (``query_weight`` ...), as the reference does for checkpoints.
    """

    def __init__(self, in_features: int, out_features: int, sequence_parallel: bool = False,
                 fuse_wgrad_accumulation: bool = False, tp_group=None, tp_size: int = 1,
                 get_rng_state_tracker: Optional[Callable] = None, rng_tracker_name: Optional[str] = None,
                 init_method: Optional[Callable] = None, bias: bool = True, return_bias: bool = False,
                 params_dtype: Optional[torch.dtype] = None, parallel_mode: Optional[str] = None,
                 parameters_split: Optional[Union[Tuple[str, ...], Dict[str, int]]] = None,
                 device: Union[torch.device, str] = None, ub_overlap_ag: bool = False, ub_overlap_rs: bool = False,
                 ub_overlap_rs_dgrad: bool = False, ub_bulk_dgrad: bool = False, ub_bulk_wgrad: bool = False,
                 ub_name: Optional[str] = None, delay_wgrad_compute: bool = False,
                 symmetric_ar_type: Optional[str] = None, save_original_input: bool = False,
                 name: Optional[str] = None) -> None:
        super().__init__()
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.in_features, self.out_features = in_features, out_features
        self.use_bias, self.return_bias = bias, return_bias
        self.apply_bias = bias and not return_bias
        self.fuse_wgrad_accumulation = fuse_wgrad_accumulation
        self.get_rng_state_tracker, self.rng_tracker_name = get_rng_state_tracker, rng_tracker_name
        self.name = name
        self.ub_name = ub_name
        # ub_* requests: in this library the collectives are fused into the GEMM kernels for every tensor-parallel
        # module once ``initialize_ub(tp_group=...)`` was called (bulk overlap of the wgrad operands included);
        # a request without that call is reported at the first forward
        self.ub_overlap_ag, self.ub_overlap_rs = ub_overlap_ag, ub_overlap_rs
        self._ub_requested = any((ub_overlap_ag, ub_overlap_rs, ub_overlap_rs_dgrad, ub_bulk_dgrad, ub_bulk_wgrad))
        if symmetric_ar_type is not None:
            raise NotImplementedError("symmetric_ar_type: the symmetric-memory all-reduce variants are not built; "
                                      "tensor-parallel all-reduces use NCCL or, with sequence parallelism, the "
                                      "fused reduce-scatter kernels")
        self.symmetric_ar_type = None
        self.save_original_input = save_original_input
        if tp_group is None:
            self.tp_size = tp_size
            if tp_size == 1:
                self.set_tensor_parallel_group(tp_group)
        else:
            self.set_tensor_parallel_group(tp_group)
        assert parallel_mode in (None, "column", "row"), f"parallel_mode {parallel_mode} not supported"
        self.parallel_mode = parallel_mode
        if parallel_mode == "column":
            assert out_features % self.tp_size == 0
            self.out_features = out_features // self.tp_size
        elif parallel_mode == "row":
            assert in_features % self.tp_size == 0
            self.in_features = in_features // self.tp_size
        self.sequence_parallel = (self.tp_size > 1) and sequence_parallel
        self.wgrad_store = WeightGradStore(delay_wgrad_compute)
        self.activation_dtype = params_dtype
        init_method = init_method or get_default_init_method()

        # parameter layout
        if parameters_split is None:
            names, sizes = ("",), (self.out_features,)
        elif isinstance(parameters_split, dict):
            names = tuple(f"{k}_" for k in parameters_split)
            sizes = tuple(parameters_split.values())
            if parallel_mode == "column":
                sizes = tuple(s // self.tp_size for s in sizes)
        else:
            names = tuple(f"{k}_" for k in parameters_split)
            assert self.out_features % len(names) == 0
            sizes = (self.out_features // len(names),) * len(names)
        assert sum(sizes) == self.out_features, "parameters_split does not add up to out_features"
        self.weight_names = [f"{n}weight" for n in names]
        self.bias_names = [f"{n}bias" for n in names]
        self._split_sizes = sizes
        weight_tensor = torch.empty(self.out_features, self.in_features, device=device, dtype=params_dtype)
        bias_tensor = torch.zeros(self.out_features, device=device, dtype=params_dtype) if bias else None
        off = 0
        for n, s in zip(names, sizes):
            w = weight_tensor[off:off + s]
            if device != "meta" and str(device) != "meta":
                self._init_weight(w, init_method)
            p = torch.nn.Parameter(w)
            if parallel_mode is not None:
                D.set_tensor_model_parallel_attributes(p, True, 0 if parallel_mode == "column" else 1, 1)
            self.register_parameter(f"{n}weight", p)
            if bias:
                bp = torch.nn.Parameter(bias_tensor[off:off + s])
                if parallel_mode == "column":
                    D.set_tensor_model_parallel_attributes(bp, True, 0, 1)
                if parallel_mode == "row" and self.sequence_parallel:
                    setattr(bp, "sequence_parallel", True)
                self.register_parameter(f"{n}bias", bp)
            off += s
        self._fused_weight_storage = weight_tensor if len(names) > 1 else None
        self._fused_bias_storage = bias_tensor if (len(names) > 1 and bias) else None
        tracker, tracker_name = get_rng_state_tracker, rng_tracker_name

        def init_w(w, f=init_method):
            if tracker is not None and parallel_mode is not None:
                with (tracker().fork(tracker_name) if tracker_name else tracker().fork()):
                    return f(w)
            return f(w)

        self._init_fns = {n: init_w for n in self.weight_names}
        if bias:
            self._init_fns.update({n: torch.nn.init.zeros_ for n in self.bias_names})
        if self.primary_weights_in_fp8:
            self._quantize_primary_weights(self.weight_names)
            self._fused_weight_storage = None
        self.cfg = F.LinearConfig(parallel_mode=self.parallel_mode, sequence_parallel=self.sequence_parallel,
                                  tp_group=self.tp_group, tp_size=self.tp_size,
                                  fuse_wgrad_accumulation=fuse_wgrad_accumulation,
                                  activation_dtype=params_dtype, wgrad_store=self.wgrad_store, name=name or "")

    def _init_weight(self, w, init_method):
        if self.get_rng_state_tracker is not None and self.parallel_mode is not None:
            tracker = self.get_rng_state_tracker()
            with (tracker.fork(self.rng_tracker_name) if self.rng_tracker_name else tracker.fork()):
                init_method(w)
        else:
            init_method(w)

    def set_tensor_parallel_group(self, tp_group) -> None:
        super().set_tensor_parallel_group(tp_group)
        if hasattr(self, "cfg"):
            self.cfg.tp_group, self.cfg.tp_size = self.tp_group, self.tp_size

    # ------------------------------------------------------------------
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

    def quantize_full_weight(self, full: torch.Tensor, dtype):
        """Quantize (or cast) a freshly assembled full weight of a distributed parameter; not cached."""
        q = self.get_quantizer(True, 1)
        if q is None:
            return full if full.dtype == dtype else full.to(dtype)
        q.set_usage(rowwise=True, columnwise=True)
        q.internal = True
        return q(full)

    def forward(self, inp: torch.Tensor, is_first_microbatch: Optional[bool] = None, fp8_output: bool = False,
                fp8_grad: bool = False):
        if fp8_output or fp8_grad:
            raise NotImplementedError("fp8_output / fp8_grad: quantized layer outputs and input gradients are not "
                                      "implemented; the next layer quantizes its own input")
        if self._ub_requested:
            from ..parallel import comm_gemm

            if self.tp_size > 1 and not comm_gemm.enabled_for(self.tp_group):
                import warnings

                warnings.warn("ub_overlap_* / ub_bulk_* was requested but initialize_ub(tp_group=...) has not been "
                              "called: the collectives of this module run on NCCL")
            self._ub_requested = False
        self.prepare_forward(num_gemms=1)
        if inp.dtype in (torch.bfloat16, torch.float16, torch.float32) and torch.is_autocast_enabled():
            self.cfg.activation_dtype = torch.get_autocast_gpu_dtype()
        else:
            self.cfg.activation_dtype = self.activation_dtype if not isinstance(inp, QuantizedTensorStorage) else inp._dtype
        if inp.is_floating_point() and not isinstance(inp, QuantizedTensorStorage) and not torch.is_autocast_enabled():
            self.cfg.activation_dtype = inp.dtype
        weight, bias = self._get_weight_bias()
        if DW.is_distributed_weight(weight):
            wq = self.quantize_full_weight(DW.materialize_weight_for_forward(weight)[0].detach(),
                                           self.cfg.activation_dtype)
        else:
            wq = self.get_quantized_weight(weight, self.get_quantizer(True, 1), cache_name="weight",
                                           is_first_microbatch=is_first_microbatch,
                                           need_columnwise=torch.is_grad_enabled() and inp.requires_grad or True)
        if isinstance(wq, torch.Tensor) and not isinstance(wq, QuantizedTensorStorage) and wq.dtype != self.cfg.activation_dtype:
            wq = wq.to(self.cfg.activation_dtype)
        b_use = bias if self.apply_bias else None
        if b_use is not None and b_use.dtype != self.cfg.activation_dtype:
            b_use = b_use.to(self.cfg.activation_dtype)
        out = _Linear.apply(inp, weight, b_use, self, self.cfg, is_first_microbatch, fp8_output, wq)
        if self.return_bias:
            return out, (bias.to(self.cfg.activation_dtype) if bias is not None else None)
        return out


class _ConcatView(torch.autograd.Function):
    """Present parameters that are views of one buffer as the whole buffer, and split the
    gradient back without a copy of the weights."""

    @staticmethod
    def forward(ctx, storage, *parts):  # type: ignore[override]
        ctx.sizes = [p.shape[0] for p in parts]
        return storage.detach()

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        return (None,) + tuple(torch.split(grad, ctx.sizes, dim=0))
