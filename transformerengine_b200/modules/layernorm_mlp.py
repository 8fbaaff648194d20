"""``LayerNormMLP``: norm -> fc1 -> activation -> fc2 in one autograd node.

Every intermediate that a GEMM reads is produced directly in the GEMM's
quantized format by a fused kernel: norm+quantize for fc1's input,
activation+quantize for fc2's input, activation-gradient+quantize(+dbias) for
fc1's dgrad/wgrad input.  Parameters: ``layer_norm_weight``,
``layer_norm_bias``, ``fc1_weight``, ``fc1_bias``, ``fc2_weight``, ``fc2_bias``;
gated activations make ``fc1_weight`` ``[2*ffn, hidden]`` with the gate rows
first (reference: ``pytorch/module/layernorm_mlp.py:174-2141``).
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch

from .. import ops
from ..parallel import distributed as D
from ..quantization import FP8GlobalStateManager
from ..tensor.base import QuantizedTensorStorage, prepare_for_saving, restore_from_saved
from . import _functional as F
from .base import TransformerEngineBaseModule, WeightGradStore, get_default_init_method


class _LayerNormMLP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, ln_w, ln_b, fc1_w, fc1_b, fc2_w, fc2_b, module, w1q, w2q, return_ln_out):  # type: ignore[override]
        cfg1, cfg2 = module.cfg1, module.cfg2
        adt = cfg1.activation_dtype
        hidden = inp.shape[-1]
        x2d = inp.reshape(-1, hidden)
        if x2d.dtype != adt:
            x2d = x2d.to(adt)
        x2d = x2d.contiguous()
        fp8 = module.fp8
        grad = any(ctx.needs_input_grad)
        q_in1, q_in2 = module.get_quantizer(True, 0), module.get_quantizer(True, 3)
        sp = cfg1.sequence_parallel and cfg1.tp_size > 1
        # recipe.backward_override: quantized forward, unquantized backward GEMMs on the original ("high_precision")
        # or on the dequantized forward operands ("dequantized")
        override = module.backward_override() if (fp8 and grad) else None
        hp_bwd = override == "high_precision"
        sp_fused_q = sp and isinstance(q_in1, F.MXFP8Quantizer) and F._fused_comm_ok(cfg1, x2d.shape[0], x2d) \
            and x2d.shape[0] % 128 == 0 and override is None
        if q_in1 is not None:
            q_in1.set_usage(rowwise=True, columnwise=grad and (not sp or sp_fused_q) and override is None)
            q_in1.internal = True
        is_ln = module.normalization == "LayerNorm"
        ln_hp, ln_q, mu, rs = ops.norm_fwd(x2d, ln_w, ln_b, module.eps, module.zero_centered_gamma, is_ln,
                                           quantizer=q_in1 if (not sp or sp_fused_q) else None,
                                           want_hp=return_ln_out or q_in1 is None or (sp and not sp_fused_q) or hp_bwd)
        act = module.activation
        fc1_out = None
        ln_total = None
        ln_local = ln_q if (sp_fused_q and ln_q is not None) else ln_hp
        if sp:
            if override is None and F._fused_comm_ok(cfg1, x2d.shape[0], x2d):
                res = F.fused_all_gather_gemm(ln_local, F.as_operand(w1q, "rowwise"), fc1_b, cfg1, q_in1, adt, "fprop",
                                              columnwise=grad)
                if res is not None:
                    fc1_out, ln_local = res[0], res[1]
            if fc1_out is None:
                ln_total = F.gather_input(ln_local, cfg1, q_in1, True, grad and override is None)
        else:
            ln_total = ln_q if ln_q is not None else ln_hp
        if fc1_out is None:
            fc1_out, _ = F.linear_fprop(ln_total, w1q, fc1_b, cfg1, adt)
        if q_in2 is not None:
            q_in2.set_usage(rowwise=True, columnwise=grad and override is None)
            q_in2.internal = True
        act_hp, act_q = ops.activation_fwd(fc1_out, act, quantizer=q_in2, want_hp=q_in2 is None or hp_bwd,
                                           params=module.activation_params)
        act_in = act_q if act_q is not None else act_hp
        out, _ = F.linear_fprop(act_in, w2q, fc2_b, cfg2, adt)
        if grad:
            keep_ln = ln_local if sp else ln_total
            if hp_bwd:
                keep_ln, act_in = ln_hp, act_hp
            elif override == "dequantized" and sp:
                keep_ln = F.quantize_for_gemm(ln_hp, q_in1, True, False)    # this rank's rows as the forward saw them
            if F._is_q(keep_ln) and keep_ln.get_usages()["columnwise"]:
                keep_ln.update_usage(rowwise_usage=False)
            if F._is_q(act_in) and act_in.get_usages()["columnwise"]:
                act_in.update_usage(rowwise_usage=False)
            ctx.w1q = w1q if F._is_q(w1q) else None  # cached objects shared across calls: not stripped
            ctx.w2q = w2q if F._is_q(w2q) else None
            flat, objs = prepare_for_saving(keep_ln, act_in)
            ctx.save_for_backward(*flat, x2d, ln_w, ln_b, mu, rs, fc1_out, fc1_w, fc1_b, fc2_w, fc2_b)
            ctx.objs = objs
            ctx.module, ctx.fp8 = module, fp8 and override is None
            ctx.override = override
            ctx.inp_shape = inp.shape
            ctx.sp = sp
            ctx.return_ln_out = return_ln_out
            ctx.reduce_bwd_amax = FP8GlobalStateManager.is_first_fp8_module() if fp8 else False
        out = out.reshape(*inp.shape[:-1], out.shape[-1]) if not sp else out.reshape(-1, *inp.shape[1:-1], out.shape[-1])
        if return_ln_out:
            return out, ln_hp.reshape(inp.shape)
        return out

    @staticmethod
    def backward(ctx, grad_output, *extra):  # type: ignore[override]
        saved = list(ctx.saved_tensors)
        fc2_b = saved.pop(); fc2_w = saved.pop(); fc1_b = saved.pop(); fc1_w = saved.pop()
        fc1_out = saved.pop(); rs = saved.pop(); mu = saved.pop(); ln_b = saved.pop(); ln_w = saved.pop()
        x2d = saved.pop()
        keep_ln, act_in = restore_from_saved(ctx.objs, saved)
        w1q, w2q = ctx.w1q, ctx.w2q
        module = ctx.module
        cfg1, cfg2 = module.cfg1, module.cfg2
        adt = cfg1.activation_dtype
        w1 = w1q if w1q is not None else fc1_w
        w2 = w2q if w2q is not None else fc2_w
        if ctx.override is not None:
            hp = lambda t: t.dequantize(dtype=adt) if F._is_q(t) else (t if t.dtype == adt else t.to(adt))  # noqa: E731
            w1, w2 = (hp(fc1_w), hp(fc2_w)) if ctx.override == "high_precision" else (hp(w1), hp(w2))
            keep_ln, act_in = hp(keep_ln), hp(act_in)
        dy2d = grad_output.reshape(-1, grad_output.shape[-1]).to(adt).contiguous()
        q_go2 = module.get_quantizer(False, 2) if ctx.fp8 else None
        q_go1 = module.get_quantizer(False, 0) if ctx.fp8 else None
        db2 = F.bias_grad(dy2d, fc2_b.dtype) if fc2_b is not None else None
        dact = None
        if ctx.sp:
            dyq, dact = F.row_parallel_grad_output(dy2d, w2, cfg2, q_go2, True, True, adt)
        else:
            dyq = F.quantize_for_gemm(dy2d, q_go2, True, True)
        # fc2 dgrad (row-parallel: no collective after dgrad) and wgrad
        if dact is None:
            dact, _, _ = F.linear_dgrad(dyq, w2, cfg2, adt)
        dw2 = F.linear_wgrad(dyq, act_in, fc2_w, cfg2) if fc2_w.requires_grad else None
        # activation backward fused with quantization (+ fc1 bias gradient)
        if q_go1 is not None:
            q_go1.set_usage(rowwise=True, columnwise=True)
            q_go1.internal = True
        dfc1_hp, dfc1_q, db1 = ops.activation_bwd(dact, fc1_out, module.activation, params=module.activation_params,
                                                  quantizer=q_go1,
                                                  want_hp=q_go1 is None, want_dbias=fc1_b is not None)
        dfc1 = dfc1_q if dfc1_q is not None else dfc1_hp
        if db1 is not None:
            db1 = db1.to(fc1_b.dtype)
        dln, h, x_total = F.linear_dgrad(dfc1, w1, cfg1, adt, async_comm=True,
                                         side=keep_ln if (ctx.sp and fc1_w.requires_grad) else None)
        dw1 = None
        if fc1_w.requires_grad:
            xw = keep_ln
            if ctx.sp:
                q_in1 = module.get_quantizer(True, 0) if ctx.fp8 else None
                xw = F.gathered_wgrad_input(keep_ln, x_total, cfg1, q_in1)
            dw1 = F.linear_wgrad(dfc1, xw, fc1_w, cfg1)
        if h is not None:
            h.wait()
        if ctx.return_ln_out and extra and extra[0] is not None:
            dln = dln + extra[0].reshape(dln.shape).to(dln.dtype)
        dx, dg, dbeta = ops.norm_bwd(dln, x2d, mu, rs, ln_w, module.zero_centered_gamma,
                                     module.normalization == "LayerNorm")
        if ctx.fp8 and ctx.reduce_bwd_amax:
            FP8GlobalStateManager.reduce_and_update_fp8_tensors(forward=False)
        return dx.reshape(ctx.inp_shape), dg, dbeta, dw1, db1, dw2, db2, None, None, None, None


class LayerNormMLP(TransformerEngineBaseModule):
    def __init__(self, hidden_size: int, ffn_hidden_size: int, eps: float = 1e-5, sequence_parallel: bool = False,
                 return_bias: bool = False, get_rng_state_tracker: Optional[Callable] = None, tp_group=None,
                 tp_size: int = 1, init_method: Optional[Callable] = None, bias: bool = True,
                 normalization: str = "LayerNorm", activation: str = "gelu", activation_params: Optional[dict] = None,
                 output_layer_init_method: Optional[Callable] = None, fuse_wgrad_accumulation: bool = False,
                 params_dtype: Optional[torch.dtype] = None, return_layernorm_output: bool = False,
                 return_layernorm_output_gathered: bool = False, seq_length: Optional[int] = None,
                 micro_batch_size: Optional[int] = None, set_parallel_mode: bool = False,
                 zero_centered_gamma: bool = False, device: Union[torch.device, str] = None,
                 ub_overlap_ag: bool = False, ub_overlap_rs: bool = False, ub_overlap_rs_dgrad: bool = False,
                 ub_bulk_dgrad: bool = False, ub_bulk_wgrad: bool = False, delay_wgrad_compute: bool = False,
                 symmetric_ar_type: Optional[str] = None, checkpoint: bool = False, name: Optional[str] = None):
        super().__init__()
        if activation_params and activation != "clamped_swiglu":
            raise NotImplementedError(f"activation_params are the limit / alpha / glu_linear_offset of "
                                      f"activation='clamped_swiglu'; activation={activation!r} takes none")
        if activation_params and set(activation_params) - {"limit", "alpha", "glu_linear_offset"}:
            raise ValueError(f"unknown activation_params {sorted(activation_params)}")
        self.activation_params = dict(activation_params) if activation_params else None
        # with sequence parallelism: return all rows of the normalized output (gathered over the tensor-parallel
        # group; gradients reduce-scatter back) instead of this rank's rows
        self.return_layernorm_output_gathered = return_layernorm_output_gathered
        if symmetric_ar_type is not None:
            raise NotImplementedError("symmetric_ar_type: use te.initialize_ub (fused GEMM + collective kernels) instead")
        if checkpoint:
            import warnings

            warnings.warn("LayerNormMLP(checkpoint=True): selective recompute inside the module is not implemented; "
                          "wrap the module in te.checkpoint to trade compute for memory", stacklevel=2)
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        assert normalization in ("LayerNorm", "RMSNorm")
        self.hidden_size, self.eps = hidden_size, eps
        self.normalization, self.zero_centered_gamma = normalization, zero_centered_gamma
        self.activation = activation
        self.use_bias, self.return_bias = bias, return_bias
        self.apply_bias = bias and not return_bias
        self.return_layernorm_output = return_layernorm_output
        self.fuse_wgrad_accumulation = fuse_wgrad_accumulation
        self.set_parallel_mode = set_parallel_mode
        self.name = name
        if tp_group is None:
            self.tp_size = tp_size
            if tp_size == 1:
                self.set_tensor_parallel_group(tp_group)
        else:
            self.set_tensor_parallel_group(tp_group)
        self.sequence_parallel = (self.tp_size > 1) and sequence_parallel
        self.size_per_partition = ffn_hidden_size // self.tp_size if set_parallel_mode else ffn_hidden_size
        self.wgrad_store = WeightGradStore(delay_wgrad_compute)
        init_method = init_method or get_default_init_method()
        output_layer_init_method = output_layer_init_method or get_default_init_method()
        gated = ops.is_gated(activation)
        fc1_out = self.size_per_partition * (2 if gated else 1)
        ln_init = torch.zeros if zero_centered_gamma else torch.ones
        self.layer_norm_weight = torch.nn.Parameter(ln_init(hidden_size, device=device, dtype=params_dtype))
        setattr(self.layer_norm_weight, "sequence_parallel", self.sequence_parallel)
        if normalization == "LayerNorm":
            self.layer_norm_bias = torch.nn.Parameter(torch.zeros(hidden_size, device=device, dtype=params_dtype))
            setattr(self.layer_norm_bias, "sequence_parallel", self.sequence_parallel)
        else:
            self.layer_norm_bias = None

        def make(shape, init):
            t = torch.empty(*shape, device=device, dtype=params_dtype)
            if str(device) != "meta":
                if get_rng_state_tracker is not None and set_parallel_mode:
                    with get_rng_state_tracker().fork():
                        init(t)
                else:
                    init(t)
            return torch.nn.Parameter(t)

        self.fc1_weight = make((fc1_out, hidden_size), init_method)
        self.fc2_weight = make((hidden_size, self.size_per_partition), output_layer_init_method)
        if set_parallel_mode:
            D.set_tensor_model_parallel_attributes(self.fc1_weight, True, 0, 1)
            D.set_tensor_model_parallel_attributes(self.fc2_weight, True, 1, 1)
        if bias:
            self.fc1_bias = torch.nn.Parameter(torch.zeros(fc1_out, device=device, dtype=params_dtype))
            self.fc2_bias = torch.nn.Parameter(torch.zeros(hidden_size, device=device, dtype=params_dtype))
            if set_parallel_mode:
                D.set_tensor_model_parallel_attributes(self.fc1_bias, True, 0, 1)
                if self.sequence_parallel:
                    setattr(self.fc2_bias, "sequence_parallel", True)
        else:
            self.fc1_bias = self.fc2_bias = None
        def init_with(f):
            def run(w):
                if get_rng_state_tracker is not None and set_parallel_mode:
                    with get_rng_state_tracker().fork():
                        return f(w)
                return f(w)
            return run

        self._init_fns = {"layer_norm_weight": torch.nn.init.zeros_ if zero_centered_gamma else torch.nn.init.ones_,
                          "fc1_weight": init_with(init_method), "fc2_weight": init_with(output_layer_init_method)}
        if normalization == "LayerNorm":
            self._init_fns["layer_norm_bias"] = torch.nn.init.zeros_
        if bias:
            self._init_fns.update(fc1_bias=torch.nn.init.zeros_, fc2_bias=torch.nn.init.zeros_)
        if self.primary_weights_in_fp8:
            self._quantize_primary_weights(("fc1_weight", "fc2_weight"))
        mode1 = "column" if set_parallel_mode else None
        mode2 = "row" if set_parallel_mode else None
        self.cfg1 = F.LinearConfig(parallel_mode=mode1, sequence_parallel=self.sequence_parallel,
                                   tp_group=self.tp_group, tp_size=self.tp_size,
                                   fuse_wgrad_accumulation=fuse_wgrad_accumulation, activation_dtype=params_dtype,
                                   wgrad_store=self.wgrad_store, name="fc1")
        self.cfg2 = F.LinearConfig(parallel_mode=mode2, sequence_parallel=self.sequence_parallel,
                                   tp_group=self.tp_group, tp_size=self.tp_size,
                                   fuse_wgrad_accumulation=fuse_wgrad_accumulation, activation_dtype=params_dtype,
                                   wgrad_store=self.wgrad_store, name="fc2")

    def set_tensor_parallel_group(self, tp_group) -> None:
        super().set_tensor_parallel_group(tp_group)
        for c in (getattr(self, "cfg1", None), getattr(self, "cfg2", None)):
            if c is not None:
                c.tp_group, c.tp_size = self.tp_group, self.tp_size

    def forward(self, inp: torch.Tensor, is_first_microbatch: Optional[bool] = None):
        self.prepare_forward(num_gemms=2)
        adt = torch.get_autocast_gpu_dtype() if torch.is_autocast_enabled() else inp.dtype
        self.cfg1.activation_dtype = self.cfg2.activation_dtype = adt
        w1q = self.get_quantized_weight(self.fc1_weight, self.get_quantizer(True, 1), cache_name="fc1_weight",
                                        is_first_microbatch=is_first_microbatch)
        w2q = self.get_quantized_weight(self.fc2_weight, self.get_quantizer(True, 4), cache_name="fc2_weight",
                                        is_first_microbatch=is_first_microbatch)
        if not isinstance(w1q, QuantizedTensorStorage) and w1q.dtype != adt:
            w1q, w2q = w1q.to(adt), w2q.to(adt)
        cast = lambda t: t.to(adt) if (t is not None and t.dtype != adt) else t  # noqa: E731
        fc1_b = cast(self.fc1_bias) if self.use_bias else None
        fc2_b = cast(self.fc2_bias) if self.apply_bias else None
        ln_w, ln_b = self.layer_norm_weight, self.layer_norm_bias
        if ln_w.dtype not in (adt, torch.float32):
            ln_w, ln_b = cast(ln_w), cast(ln_b)
        res = _LayerNormMLP.apply(inp, ln_w, ln_b, self.fc1_weight, fc1_b, self.fc2_weight, fc2_b, self, w1q, w2q,
                                  self.return_layernorm_output)
        out, ln_out = (res if self.return_layernorm_output else (res, None))
        if ln_out is not None and self.return_layernorm_output_gathered and self.cfg1.sequence_parallel \
                and self.cfg1.tp_size > 1:
            from ..parallel.distributed import gather_rows_with_grad
            ln_out = gather_rows_with_grad(ln_out, self.cfg1.tp_group)
        if self.return_bias:
            fb = cast(self.fc2_bias) if self.use_bias else None
            if self.return_layernorm_output:
                return out, fb, ln_out
            return out, fb
        if self.return_layernorm_output:
            return out, ln_out
        return out
