"""``GroupedLinear``: ``num_gemms`` independent linear layers applied to consecutive row slabs
of one input (MoE experts), and ``Fp8Padding`` / ``Fp8Unpadding`` that align the slabs for
quantized GEMMs (reference: ``pytorch/module/grouped_linear.py:154-2137``,
``fp8_padding.py``, ``fp8_unpadding.py``).

Forward and dgrad of all groups run as ONE launch of the tcgen05 grouped GEMM (device-side
slab offsets) when the slabs are 128-row aligned; otherwise, and for wgrad (contraction over
the rows of a slab), one GEMM per group is issued.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Union

import torch

from .. import ops
from ..ops.gemm import Operand, as_operand, gemm_nt
from ..quantization import FP8GlobalStateManager, get_align_size_for_quantization
from ..tensor.base import QuantizedTensorStorage
from ..tensor.mxfp8 import MXFP8Quantizer
from . import _functional as F
from .base import TransformerEngineBaseModule, WeightGradStore, get_default_init_method


_OFFSET_CACHE: dict = {}


def _offsets(m_splits: List[int], device) -> torch.Tensor:
    """Row offsets of the slabs as an int32 device tensor; the last few are kept (a forward and its backward ask
    for the same offsets several times, each miss is a host-to-device copy)."""
    key = (tuple(int(m) for m in m_splits), str(device))
    t = _OFFSET_CACHE.get(key)
    if t is None:
        offs = [0]
        for m in key[0]:
            offs.append(offs[-1] + m)
        t = torch.tensor(offs, dtype=torch.int32, device=device)
        if len(_OFFSET_CACHE) >= 64:
            _OFFSET_CACHE.pop(next(iter(_OFFSET_CACHE)))
        _OFFSET_CACHE[key] = t
    return t


def _can_group(m_splits, x_ops, quantized: bool) -> bool:
    if not getattr(x_ops.data, "is_cuda", False):
        return False
    if quantized:
        return all(m % 128 == 0 for m in m_splits)
    return True


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, m_splits, module, adt, *weights_and_biases):  # type: ignore[override]
        G = module.num_gemms
        weights = list(weights_and_biases[:G])
        biases = list(weights_and_biases[G:]) if module.use_bias else [None] * G
        x2d = inp.reshape(-1, inp.shape[-1])
        if x2d.dtype != adt:
            x2d = x2d.to(adt)
        fp8 = module.fp8
        grad_on = any(ctx.needs_input_grad)
        N, K = module.out_features, module.in_features
        out = torch.empty(x2d.shape[0], N, dtype=adt, device=x2d.device)
        offs = [0]
        for m in m_splits:
            offs.append(offs[-1] + int(m))
        in_q = module.get_quantizer(True, 0)
        quant_ok = fp8 and in_q is not None and all(m % 32 == 0 for m in m_splits) and K % 32 == 0
        # recipe.backward_override: quantized forward, 16-bit backward GEMMs on the original ("high_precision") or the
        # dequantized forward operands ("dequantized")
        override = module.backward_override() if (quant_ok and grad_on) else None
        xq = None
        wqs = []
        if quant_ok:
            in_q.set_usage(rowwise=True, columnwise=grad_on and override is None)
            in_q.internal = True
            aligned = all(m % 128 == 0 for m in m_splits) and isinstance(in_q, MXFP8Quantizer)
            for g in range(G):
                wqs.append(module.get_quantized_weight(weights[g], module.get_quantizer(True, 3 * g + 1),
                                                       cache_name=f"weight{g}"))
            if aligned and x2d.shape[0] > 0:
                xq = in_q(x2d)  # one quantization for all slabs
                a = as_operand(xq, "rowwise")
                b = module.stacked_weight_operand(wqs, "rowwise")
                if _can_group(m_splits, a, True):
                    gemm_nt(a, b, out=out, group_offsets=_offsets(m_splits, x2d.device), num_groups=G)
                else:
                    xq = None
            if xq is None:
                xs = []
                for g in range(G):
                    if m_splits[g] == 0:
                        xs.append(None)
                        continue
                    xg = in_q(x2d[offs[g]:offs[g + 1]])
                    xs.append(xg)
                    gemm_nt(as_operand(xg, "rowwise"), as_operand(wqs[g], "rowwise"), out=out[offs[g]:offs[g + 1]])
                xq = xs
        else:
            wcat = None
            if getattr(x2d, "is_cuda", False) and x2d.shape[0] > 0 and adt in (torch.bfloat16, torch.float16):
                wcat = torch.cat([w.to(adt) for w in weights], 0)
                gemm_nt(x2d, wcat, out=out, group_offsets=_offsets(m_splits, x2d.device), num_groups=G)
            else:
                for g in range(G):
                    if m_splits[g]:
                        gemm_nt(x2d[offs[g]:offs[g + 1]], weights[g].to(adt), out=out[offs[g]:offs[g + 1]])
            xq = x2d
        if biases[0] is not None:
            # every slab gets its expert's bias: one launch for all of them
            ops.grouped_bias_add_(out, torch.stack([b.to(adt) for b in biases]), _offsets(m_splits, out.device))
        if grad_on:
            ctx.module, ctx.m_splits, ctx.offs, ctx.adt, ctx.fp8q = module, list(m_splits), offs, adt, quant_ok
            ctx.xq, ctx.wqs = (x2d if override == "high_precision" else xq), wqs
            ctx.override = override
            ctx.save_for_backward(*weights)
            ctx.inp_shape = inp.shape
            ctx.reduce_bwd_amax = FP8GlobalStateManager.is_first_fp8_module() if fp8 else False
        return out.reshape(*inp.shape[:-1], N)

    @staticmethod
    def backward(ctx, grad_out):  # type: ignore[override]
        module, m_splits, offs, adt = ctx.module, ctx.m_splits, ctx.offs, ctx.adt
        weights = list(ctx.saved_tensors)
        G, N, K = module.num_gemms, module.out_features, module.in_features
        dy = grad_out.reshape(-1, N).to(adt).contiguous()
        dx = torch.empty(dy.shape[0], K, dtype=adt, device=dy.device)
        dws = [None] * G
        dbs = [None] * G
        x_hp = None  # input dequantized ONCE when it was saved as one quantized tensor
        fp8q, xq, w_hp = ctx.fp8q, ctx.xq, None
        if ctx.override is not None:
            fp8q = False
            if ctx.override == "dequantized":
                w_hp = [wq.dequantize(dtype=adt) for wq in ctx.wqs]
                if isinstance(xq, list):      # one quantized tensor per slab (None for an empty slab)
                    pieces = xq
                    xq = torch.zeros(dy.shape[0], K, dtype=adt, device=dy.device)
                    for g, piece in enumerate(pieces):
                        if piece is not None:
                            xq[offs[g]:offs[g + 1]] = piece.dequantize(dtype=adt)
                else:
                    xq = xq.dequantize(dtype=adt)
        if fp8q and isinstance(ctx.xq, QuantizedTensorStorage) and dy.is_cuda and dy.shape[0] > 0 \
                and N % 32 == 0 and all(m % 128 == 0 for m in m_splits):
            # Slabs are whole 128-row tiles: grad_output is quantized ONCE (both copies), dgrad is one grouped
            # launch over the stacked column-wise weights, and every wgrad GEMM reads its slab as a view of the
            # column-wise copies (contraction over the slab's rows) -- nothing is dequantized or re-quantized.
            from ..ops.gemm import contraction_slab

            gq = module.get_quantizer(False, 0)
            gq.set_usage(rowwise=True, columnwise=True)
            gq.internal = True
            dyq = gq(dy)
            wcol = module.stacked_weight_operand(ctx.wqs, "columnwise")        # [G * K, N]
            gemm_nt(as_operand(dyq, "rowwise"), wcol, out=dx, group_offsets=_offsets(m_splits, dy.device), num_groups=G)
            dy_col, x_col = as_operand(dyq, "columnwise"), as_operand(ctx.xq, "columnwise")
            if module.use_bias:
                db_all = ops.grouped_column_sum(dy, _offsets(m_splits, dy.device), torch.float32)
                dbs = [db_all[g].to(weights[g].dtype) for g in range(G)]
            for g in range(G):
                if m_splits[g] == 0:
                    dws[g] = torch.zeros_like(weights[g])
                    continue
                dws[g] = _wgrad(module, weights[g], lambda a=contraction_slab(dy_col, offs[g], offs[g + 1]),
                                b=contraction_slab(x_col, offs[g], offs[g + 1]), w=weights[g]: gemm_nt(
                                    a, b, out_dtype=w.dtype if w.dtype != torch.float32 else torch.float32))
            if ctx.reduce_bwd_amax:
                FP8GlobalStateManager.reduce_and_update_fp8_tensors(forward=False)
            res = [dx.reshape(ctx.inp_shape), None, None, None] + dws
            if module.use_bias:
                res += dbs
            return tuple(res)
        if module.use_bias:
            db_all = ops.grouped_column_sum(dy, _offsets(m_splits, dy.device), torch.float32)
            dbs = [db_all[g].to(weights[g].dtype) for g in range(G)]
        for g in range(G):
            sl = slice(offs[g], offs[g + 1])
            if m_splits[g] == 0:
                dws[g] = torch.zeros_like(weights[g])
                continue
            if fp8q:
                gq = module.get_quantizer(False, 2 * g)
                gq.set_usage(rowwise=True, columnwise=True)
                gq.internal = True
                dyq = gq(dy[sl])
                xg = ctx.xq[g] if isinstance(ctx.xq, list) else None
                gemm_nt(as_operand(dyq, "rowwise"), as_operand(ctx.wqs[g], "columnwise"), out=dx[sl])
                if xg is None:
                    # the input was quantized as one tensor: re-quantize this slab's rows columnwise
                    in_q = module.get_quantizer(True, 0)
                    in_q.set_usage(rowwise=False, columnwise=True)
                    if isinstance(ctx.xq, QuantizedTensorStorage):
                        if x_hp is None:
                            x_hp = ctx.xq.dequantize(dtype=adt)
                        xg = in_q(x_hp[sl])
                    else:
                        xg = in_q(ctx.xq[sl])
                dws[g] = _wgrad(module, weights[g], lambda a=as_operand(dyq, "columnwise"),
                                b=as_operand(xg, "columnwise"), w=weights[g]: gemm_nt(
                                    a, b, out_dtype=w.dtype if w.dtype != torch.float32 else torch.float32))
            else:
                w = w_hp[g] if w_hp is not None else weights[g].to(adt)
                gemm_nt(as_operand(dy[sl], "rowwise"), as_operand(w, "columnwise"), out=dx[sl])
                dws[g] = _wgrad(module, weights[g], lambda a=as_operand(dy[sl], "columnwise"),
                                b=as_operand(xq[sl], "columnwise"), w=weights[g]: gemm_nt(a, b, out_dtype=w.dtype))
        if fp8q and ctx.reduce_bwd_amax:
            FP8GlobalStateManager.reduce_and_update_fp8_tensors(forward=False)
        res = [dx.reshape(ctx.inp_shape), None, None, None] + dws
        if module.use_bias:
            res += dbs
        return tuple(res)


def _wgrad(module, weight, compute):
    """Run (or, with ``delay_wgrad_compute``, queue for ``backward_dw()``) one expert's weight-gradient GEMM;
    with ``fuse_wgrad_accumulation`` the result goes into ``weight.main_grad`` and nothing is returned."""
    def finish(dw):
        if module.fuse_wgrad_accumulation and hasattr(weight, "main_grad"):
            weight.main_grad.add_(dw.float())
            return None
        return dw

    store = module.wgrad_store
    if store is not None and store.delay_wgrad_compute():
        def deferred():
            dw = finish(compute())
            if dw is not None:
                weight.grad = dw if weight.grad is None else weight.grad + dw
        store.put(deferred)
        return None
    return finish(compute())


class GroupedLinear(TransformerEngineBaseModule):
    def stacked_weight_operand(self, wqs, usage: str) -> Operand:
        """All groups' quantized weights as ONE grouped-GEMM operand (rows of group g at ``[g*rows, (g+1)*rows)``).
        The concatenation is cached until the weights change (it is redone once per optimizer step)."""
        from .base import weights_epoch

        key = (usage, weights_epoch(), tuple(id(w) for w in wqs))
        ent = self._weight_cache.get(f"stacked_{usage}")
        if ent is not None and ent[0] == key:
            return ent[1]
        ops_ = [as_operand(w, usage) for w in wqs]
        op = Operand("mxfp8", torch.cat([o.data for o in ops_], 0), torch.cat([o.scale for o in ops_], 0),
                     ops_[0].fp8_dtype, rows=sum(o.rows for o in ops_), k=ops_[0].k)
        self._weight_cache[f"stacked_{usage}"] = (key, op, None, None)
        return op

    def __init__(self, num_gemms: int, in_features: int, out_features: int, sequence_parallel: bool = False,
                 fuse_wgrad_accumulation: bool = False, tp_group=None, tp_size: int = 1,
                 get_rng_state_tracker: Optional[Callable] = None, rng_tracker_name: Optional[str] = None,
                 init_method: Optional[Callable] = None, bias: bool = True, return_bias: bool = False,
                 params_dtype: Optional[torch.dtype] = None, parallel_mode: Optional[str] = None,
                 device: Union[torch.device, str] = None, ub_overlap_rs: bool = False, ub_overlap_ag: bool = False,
                 ub_name: Optional[str] = None, delay_wgrad_compute: bool = False,
                 save_original_input: bool = False, single_grouped_weight: bool = False,
                 single_grouped_bias: bool = False, use_grouped_tensor: Optional[bool] = None,
                 name: Optional[str] = None) -> None:
        super().__init__()
        # accepted for compatibility: there is one path here, a grouped GEMM over the stacked expert operands
        # (what the reference selects with use_grouped_tensor=True), for discrete weight{i} parameters
        if use_grouped_tensor is not None and not isinstance(use_grouped_tensor, bool):
            raise TypeError(f"use_grouped_tensor must be a bool or None, got {type(use_grouped_tensor)}")
        self.use_grouped_tensor = True if use_grouped_tensor is None else use_grouped_tensor
        # options of the reference that this module does not implement are refused, not ignored
        for opt, val in (("save_original_input", save_original_input),
                         ("single_grouped_weight", single_grouped_weight), ("single_grouped_bias", single_grouped_bias)):
            if val:
                raise NotImplementedError(f"GroupedLinear({opt}=True) is not implemented")
        if ub_overlap_rs or ub_overlap_ag:
            raise NotImplementedError("GroupedLinear has no fused collective path (ub_overlap_*)")
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.num_gemms = num_gemms
        self.wgrad_store = WeightGradStore(delay_wgrad_compute)
        self.use_bias, self.return_bias = bias, return_bias
        self.apply_bias = bias and not return_bias
        self.fuse_wgrad_accumulation = fuse_wgrad_accumulation
        self.name = name
        if tp_group is None:
            self.tp_size = tp_size
        else:
            self.set_tensor_parallel_group(tp_group)
        self.parallel_mode = parallel_mode
        assert parallel_mode in (None, "column", "row")
        if parallel_mode == "column":
            out_features //= self.tp_size
        elif parallel_mode == "row":
            in_features //= self.tp_size
        self.in_features, self.out_features = in_features, out_features
        init_method = init_method or get_default_init_method()
        # all expert weights live in one [G * out, in] buffer; weight{i} are views of it
        self._stacked = torch.empty(num_gemms * out_features, in_features, device=device, dtype=params_dtype)
        for i in range(num_gemms):
            w = self._stacked[i * out_features:(i + 1) * out_features]
            if str(device) != "meta":
                init_method(w)
            self.register_parameter(f"weight{i}", torch.nn.Parameter(w))
            if bias:
                self.register_parameter(f"bias{i}", torch.nn.Parameter(
                    torch.zeros(out_features, device=device, dtype=params_dtype)))
        self._init_fns = {f"weight{i}": init_method for i in range(num_gemms)}
        if bias:
            self._init_fns.update({f"bias{i}": torch.nn.init.zeros_ for i in range(num_gemms)})
        if self.primary_weights_in_fp8:
            self._quantize_primary_weights([f"weight{i}" for i in range(num_gemms)])
            self._stacked = None

    def forward(self, inp: torch.Tensor, m_splits: List[int], is_first_microbatch: Optional[bool] = None,
                out: Optional[torch.Tensor] = None, dgrad_out: Optional[torch.Tensor] = None):
        """``out`` / ``dgrad_out``: caller-owned buffers ``[tokens, out_features]`` / ``[tokens, in_features]``
        (2-D, contiguous, not requiring grad, activation dtype) that receive the forward output and the input
        gradient; the returned tensor (and the gradient autograd hands on) are views of them.  Only the first
        ``sum(m_splits)`` rows are written.  The results are copied into the buffers (one extra pass each)."""
        if out is not None or dgrad_out is not None:
            rows = int(sum(m_splits))
            for name, buf, width in (("out", out, self.out_features), ("dgrad_out", dgrad_out, self.in_features)):
                if buf is None:
                    continue
                if buf.dim() != 2 or not buf.is_contiguous() or buf.requires_grad or buf.shape[1] != width \
                        or buf.shape[0] < rows:
                    raise ValueError(f"{name} must be a contiguous 2-D tensor without grad of shape "
                                     f"[>= {rows}, {width}], got {tuple(buf.shape)}")
            if dgrad_out is not None and inp.requires_grad:
                inp = _GradInto.apply(inp, dgrad_out, rows)
            res = self.forward(inp, m_splits, is_first_microbatch)
            if out is None:
                return res
            y, rest = (res[0], res[1:]) if isinstance(res, tuple) else (res, ())
            if y.dtype != out.dtype:
                raise ValueError(f"out has dtype {out.dtype}, the layer computes in {y.dtype}")
            out[:rows].copy_(y[:rows])
            return (out,) + tuple(rest) if rest else out
        assert len(m_splits) == self.num_gemms, "one row count per GEMM"
        self.prepare_forward(num_gemms=self.num_gemms)
        adt = torch.get_autocast_gpu_dtype() if torch.is_autocast_enabled() else inp.dtype
        ws = [getattr(self, f"weight{i}") for i in range(self.num_gemms)]
        bs = [getattr(self, f"bias{i}") for i in range(self.num_gemms)] if self.use_bias else []
        if not self.apply_bias and self.use_bias:
            out = _GroupedLinear.apply(inp, m_splits, _NoBias(self), adt, *ws)
            return out, [b.to(adt) for b in bs]
        return _GroupedLinear.apply(inp, m_splits, self, adt, *ws, *bs)


class _GradInto(torch.autograd.Function):
    """Identity whose backward writes the incoming gradient into a caller-owned buffer."""

    @staticmethod
    def forward(ctx, x, buf, rows):  # type: ignore[override]
        ctx.buf, ctx.rows = buf, rows
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        buf, rows = ctx.buf, ctx.rows
        g2 = g.reshape(-1, g.shape[-1])
        if buf.dtype != g2.dtype or g2.shape[0] > buf.shape[0]:
            return g, None, None
        buf[:rows].copy_(g2[:rows])
        return buf[:g2.shape[0]].view(g.shape), None, None


class _NoBias:
    """View of a GroupedLinear that skips the bias add (``return_bias=True``)."""

    def __init__(self, m):
        self._m = m
        self.use_bias = False

    def __getattr__(self, k):
        return getattr(self._m, k)


class Fp8Padding(torch.nn.Module):
    """Pad every row slab with zero rows up to a multiple of ``align_size``."""

    def __init__(self, num_gemms: int, align_size: Optional[int] = None) -> None:
        super().__init__()
        self.num_gemms, self.align_size = num_gemms, align_size

    def forward(self, inp: torch.Tensor, m_splits: List[int]):
        align = self.align_size or get_align_size_for_quantization(FP8GlobalStateManager.get_fp8_recipe())
        padded = [(m + align - 1) // align * align for m in m_splits]
        if padded == list(m_splits):
            return inp, list(m_splits)
        return ops.repad_rows(inp.reshape(-1, inp.shape[-1]), list(m_splits), padded), padded


class Fp8Unpadding(torch.nn.Module):
    """Inverse of :class:`Fp8Padding`."""

    def __init__(self, num_gemms: int, align_size: Optional[int] = None) -> None:
        super().__init__()
        self.num_gemms, self.align_size = num_gemms, align_size

    def forward(self, inp: torch.Tensor, m_splits: List[int]):
        align = self.align_size or get_align_size_for_quantization(FP8GlobalStateManager.get_fp8_recipe())
        padded = [(m + align - 1) // align * align for m in m_splits]
        if padded == list(m_splits):
            return inp
        return ops.repad_rows(inp.reshape(-1, inp.shape[-1]), padded, list(m_splits))
