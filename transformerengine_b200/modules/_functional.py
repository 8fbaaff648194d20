"""Shared forward/backward building blocks of the linear-family modules.

``fprop``:  ``y = x @ W^T (+ b)``            operands: x rowwise, W rowwise
``dgrad``:  ``dx = dy @ W``                  operands: dy rowwise, W columnwise
``wgrad``:  ``dW = dy^T @ x``                operands: dy columnwise, x columnwise
(reference data flow: ``pytorch/module/linear.py:268-1352``).  Tensor parallel:
column-parallel layers all-gather a sequence-sharded input before fprop and
reduce-scatter (or all-reduce) dgrad; row-parallel layers reduce-scatter (or
all-reduce) the fprop output and all-gather grad_output.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple

import torch

from .. import ops
from ..ops.gemm import as_operand, gemm_nt
from ..parallel import distributed as D
from ..tensor.base import QuantizedTensorStorage, Quantizer
from ..tensor.mxfp8 import MXFP8Quantizer, MXFP8TensorStorage


@dataclass
class LinearConfig:
    """Static settings of one GEMM of a module."""

    parallel_mode: Optional[str] = None  # None | "column" | "row"
    sequence_parallel: bool = False
    tp_group: Any = None
    tp_size: int = 1
    fuse_wgrad_accumulation: bool = False
    activation_dtype: torch.dtype = torch.float32
    wgrad_store: Any = None
    comm_overlap: Any = None  # parallel.comm_gemm.CommGemm when fused collectives are enabled
    name: str = ""


def _is_q(t) -> bool:
    return isinstance(t, QuantizedTensorStorage)


def quantize_for_gemm(x2d: torch.Tensor, quantizer: Optional[Quantizer], rowwise: bool, columnwise: bool):
    """Quantize an activation / gradient for the GEMMs that will consume it."""
    if quantizer is None or _is_q(x2d):
        return x2d
    if not quantizer.is_quantizable(x2d):
        return x2d
    quantizer.set_usage(rowwise=rowwise, columnwise=columnwise)
    quantizer.internal = True
    return quantizer(x2d)


def gather_input(x, cfg: LinearConfig, quantizer, rowwise: bool, columnwise: bool):
    """Sequence-parallel all-gather (+ quantize) of a column-parallel layer's input."""
    local_rows = x.shape[0] if not _is_q(x) else x._rows_cols()[0]
    if quantizer is not None and isinstance(quantizer, MXFP8Quantizer) and local_rows % 128 == 0:
        q = quantize_for_gemm(x, quantizer, rowwise, columnwise)
        if isinstance(q, MXFP8TensorStorage):
            return D.gather_mxfp8_along_first_dim(q, cfg.tp_group)
    if _is_q(x):
        x = x.dequantize()
    total, _ = D.gather_along_first_dim(x, cfg.tp_group)
    return quantize_for_gemm(total, quantizer, rowwise, columnwise)


def _fused_comm_ok(cfg: LinearConfig, rows_local: int, *tensors) -> bool:
    """Fused collective GEMMs need the feature switched on for this TP group, CUDA operands and
    whole 128-row blocks per rank."""
    from ..parallel import comm_gemm

    if not (cfg.sequence_parallel and cfg.tp_size > 1 and comm_gemm.enabled_for(cfg.tp_group)):
        return False
    if rows_local % 128 != 0:
        return False
    return all(getattr(as_operand(t).data, "is_cuda", False) for t in tensors)


def _comm_kind(a_op, b_op):
    """'mx', 'hp' or None when the operand pair has no fused collective kernel."""
    if a_op.kind == "mxfp8" and b_op.kind == "mxfp8" and a_op.k % 128 == 0:
        return "mx"
    if a_op.kind == "hp" and b_op.kind == "hp" and a_op.data.dtype == b_op.data.dtype \
            and a_op.data.dtype in (torch.bfloat16, torch.float16) and a_op.k % 8 == 0 \
            and a_op.data.is_contiguous() and b_op.data.is_contiguous():
        return "hp"
    return None


def _side_pack(t, world: int):
    """Describe ``t`` (this rank's rows of a wgrad operand) for the side gather of a fused kernel.
    Returns (spec, data, scales, rebuild) or None when the layout is not covered."""
    from ..parallel.comm_gemm import SideSpec

    if isinstance(t, MXFP8TensorStorage):
        cd, cs = t._columnwise_data, t._columnwise_scale_inv
        if cd is None or not cd.is_cuda:
            return None
        C, R = cd.shape
        if R % 128 != 0 or R > 32768:
            return None

        def rebuild(gd, gsf, t=t, C=C, R=R):
            return MXFP8TensorStorage(rowwise_data=None, rowwise_scale_inv=None, columnwise_data=gd.view(C, world * R),
                                      columnwise_scale_inv=gsf, fp8_dtype=t._fp8_dtype, quantizer=t._quantizer,
                                      shape=(world * R, C), dtype=t._dtype)

        return SideSpec.for_mxfp8_columnwise(C, R), cd, cs, rebuild
    if isinstance(t, torch.Tensor) and not _is_q(t) and t.is_cuda and t.dim() == 2 and t.is_contiguous() \
            and t.dtype in (torch.bfloat16, torch.float16):
        R, K = t.shape
        rb = K * t.element_size()
        if rb % 16 != 0 or rb > 32768:
            return None

        def rebuild(gd, gsf, dt=t.dtype, R=R, K=K):
            return gd.view(dt).reshape(world * R, K)

        return SideSpec.for_rows(R, rb), t, None, rebuild
    return None


def fused_all_gather_gemm(x_local, w_op, bias, cfg: LinearConfig, quantizer, out_dtype, tag: str, *,
                          columnwise: bool = False, side=None):
    """Sequence-parallel all-gather of ``x_local`` fused into ``gather(x) @ w^T``.

    ``columnwise`` also produces the column-wise copy of the local rows when they are quantized here
    (the caller keeps it for the weight gradient).  ``side`` is this rank's piece of a second operand
    that the same kernel gathers next to the GEMM (``_side_pack`` layouts).
    Returns None when this operand pair is not covered (caller falls back to NCCL + GEMM), else
    ``(out, x_local as used, gathered side or None)``."""
    from ..parallel import comm_gemm

    xq = quantize_for_gemm(x_local, quantizer, True, columnwise) if not _is_q(x_local) else x_local
    a_op = as_operand(xq, "rowwise")
    kind = _comm_kind(a_op, w_op)
    if kind is None or out_dtype not in (torch.bfloat16, torch.float16):
        return None
    T = a_op.rows * cfg.tp_size
    pack = _side_pack(side, cfg.tp_size) if side is not None else None
    ctx = comm_gemm.get_all_gather_gemm(f"{cfg.name}.{tag}", cfg.tp_group, T, a_op.k, kind == "mx",
                                        a_op.data.dtype, side=pack[0] if pack else None)
    if pack is None:
        return ctx(a_op, w_op, bias=bias, out_dtype=out_dtype), xq, None
    out, gd, gsf = ctx(a_op, w_op, bias=bias, out_dtype=out_dtype, side=(pack[1], pack[2]))
    return out, xq, pack[3](gd, gsf)


def fused_gemm_reduce_scatter(a_op, b_op, bias, cfg: LinearConfig, out_dtype, tag: str, *, side=None):
    """``reduce_scatter(a @ b^T)`` in one kernel; ``side`` as in :func:`fused_all_gather_gemm`.
    Returns None when not covered, else ``(out, gathered side or None)``."""
    from ..parallel import comm_gemm

    if _comm_kind(a_op, b_op) is None or out_dtype not in (torch.bfloat16, torch.float16):
        return None
    pack = _side_pack(side, cfg.tp_size) if side is not None else None
    ctx = comm_gemm.get_gemm_reduce_scatter(f"{cfg.name}.{tag}", cfg.tp_group, a_op.rows, b_op.rows, out_dtype,
                                            side=pack[0] if pack else None)
    if pack is None:
        return ctx(a_op, b_op, bias=bias), None
    out, gd, gsf = ctx(a_op, b_op, bias=bias, side=(pack[1], pack[2]))
    return out, pack[3](gd, gsf)


def fused_gemm_all_reduce(a_op, b_op, bias, cfg: LinearConfig, out_dtype):
    """``all_reduce(a @ b^T)`` in one kernel (row-parallel layer without sequence parallelism); None when not covered.
    The result is copied out of the kernel's double-buffered symmetric buffer, so it may be kept."""
    from ..parallel import comm_gemm

    if not (cfg.tp_size > 1 and not cfg.sequence_parallel and comm_gemm.enabled_for(cfg.tp_group)):
        return None
    if a_op.rows % (128 * cfg.tp_size) != 0 or not getattr(a_op.data, "is_cuda", False):
        return None
    if _comm_kind(a_op, b_op) is None or out_dtype not in (torch.bfloat16, torch.float16):
        return None
    ctx = comm_gemm.get_gemm_all_reduce(f"{cfg.name}.fprop", cfg.tp_group, a_op.rows, b_op.rows, out_dtype)
    return ctx(a_op, b_op, bias=bias).clone()


def linear_fprop(x, w, bias, cfg: LinearConfig, out_dtype, *, gelu: bool = False):
    """``x`` [T, in] (plain or quantized, already gathered), ``w`` [out, in].
    Returns (out2d after the row-parallel collective, pre-gelu aux or None)."""
    aux = None
    fuse_bias = bias is not None and not (cfg.parallel_mode == "row" and cfg.tp_size > 1)
    a, b = as_operand(x, "rowwise"), as_operand(w, "rowwise")
    if cfg.parallel_mode == "row" and not gelu and _fused_comm_ok(cfg, a.rows // max(cfg.tp_size, 1), x, w):
        res = fused_gemm_reduce_scatter(a, b, bias, cfg, out_dtype, "fprop")
        if res is not None:
            return res[0], None
    if cfg.parallel_mode == "row" and not gelu and not cfg.sequence_parallel and cfg.tp_size > 1:
        res = fused_gemm_all_reduce(a, b, bias, cfg, out_dtype)
        if res is not None:
            return res, None
    if gelu:
        aux = torch.empty(a.rows, b.rows, dtype=out_dtype, device=a.data.device)
        out = gemm_nt(a, b, out_dtype=out_dtype, bias=bias if fuse_bias else None, epilogue=ops.gemm.EPI_GELU, aux=aux)
    else:
        out = gemm_nt(a, b, out_dtype=out_dtype, bias=bias if fuse_bias else None)
    if cfg.parallel_mode == "row" and cfg.tp_size > 1:
        if cfg.sequence_parallel:
            out, _ = D.reduce_scatter_along_first_dim(out, cfg.tp_group)
        else:
            out, _ = D.allreduce(out, cfg.tp_group)
        if bias is not None:
            out = out + bias.to(out.dtype)
    return out, aux


def row_parallel_grad_output(dy_local, w, cfg: LinearConfig, quantizer, need_dgrad: bool, need_wgrad: bool, out_dtype):
    """Backward of a row-parallel layer under sequence parallelism: grad_output arrives sharded on
    rows.  Returns (gathered grad_output for the wgrad / dgrad GEMMs, dx or None).  With fused
    collectives the all-gather runs inside the dgrad GEMM, whose copy CTAs also gather the columnwise
    copy (the wgrad operand) while the tiles are computed."""
    if need_dgrad and _fused_comm_ok(cfg, dy_local.shape[0], dy_local):
        dq = quantize_for_gemm(dy_local, quantizer, True, need_wgrad)
        w_op = as_operand(w, "columnwise")
        if _comm_kind(as_operand(dq, "rowwise"), w_op) is not None:
            side = dq if need_wgrad and _side_pack(dq, cfg.tp_size) is not None else None
            dx, _, total = fused_all_gather_gemm(dq, w_op, None, cfg, None, out_dtype, "dgrad", side=side)
            if need_wgrad and total is None:
                if _is_q(dq):
                    import copy as _copy

                    col = _copy.copy(dq)
                    col.update_usage(rowwise_usage=False)
                    total = D.gather_mxfp8_along_first_dim(col, cfg.tp_group)
                else:
                    total, _ = D.gather_along_first_dim(dq, cfg.tp_group)
            return total, dx
    return gather_input(dy_local, cfg, quantizer, need_dgrad, need_wgrad), None


def linear_dgrad(dy, w, cfg: LinearConfig, out_dtype, *, async_comm: bool = False, side=None):
    """``dx = dy @ W``; column-parallel layers then reduce-scatter / all-reduce.

    ``side``: this rank's rows of the layer input that the weight gradient needs gathered (sequence
    parallel column-parallel layers); the fused kernel gathers it while it computes.
    Returns (dx2d, comm handle or None, gathered side or None)."""
    a, b = as_operand(dy, "rowwise"), as_operand(w, "columnwise")
    if cfg.parallel_mode == "column" and _fused_comm_ok(cfg, a.rows // max(cfg.tp_size, 1), dy):
        if side is not None and _side_pack(side, cfg.tp_size) is None:
            side = None
        res = fused_gemm_reduce_scatter(a, b, None, cfg, out_dtype, "dgrad", side=side)
        if res is not None:
            return res[0], None, res[1]
    dx = gemm_nt(a, b, out_dtype=out_dtype)
    h = None
    if cfg.parallel_mode == "column" and cfg.tp_size > 1:
        if cfg.sequence_parallel:
            dx, h = D.reduce_scatter_along_first_dim(dx, cfg.tp_group, async_op=async_comm)
        else:
            dx, h = D.allreduce(dx, cfg.tp_group, async_op=async_comm)
    return dx, h, None


def gathered_wgrad_input(keep_x, total, cfg: LinearConfig, quantizer):
    """The full-sequence wgrad operand of a sequence-parallel column-parallel layer: what the fused
    dgrad kernel gathered (quantized now if it travelled in 16 bits), else an NCCL gather."""
    if total is None:
        return gather_input(keep_x, cfg, quantizer, False, True)
    if not _is_q(total) and quantizer is not None:
        return quantize_for_gemm(total, quantizer, False, True)
    return total


def linear_wgrad(dy, x, weight: torch.Tensor, cfg: LinearConfig):
    """``dW = dy^T @ x``.  With ``fuse_wgrad_accumulation`` the product is accumulated into
    ``weight.main_grad`` (fp32) inside the GEMM epilogue and a dummy is returned."""
    a, b = as_operand(dy, "columnwise"), as_operand(x, "columnwise")

    def run():
        if cfg.fuse_wgrad_accumulation and hasattr(weight, "main_grad"):
            first = getattr(weight, "overwrite_main_grad", False) or not getattr(weight, "grad_added_to_main_grad_once", True)
            gemm_nt(a, b, out=weight.main_grad.reshape(a.rows, b.rows), accumulate=not first)
            return None
        return gemm_nt(a, b, out_dtype=weight.dtype if weight.dtype in (torch.bfloat16, torch.float16, torch.float32)
                       else cfg.activation_dtype)

    if cfg.wgrad_store is not None and cfg.wgrad_store.delay_wgrad_compute():
        def deferred():
            g = run()
            if g is not None:
                weight.grad = g if weight.grad is None else weight.grad + g
        cfg.wgrad_store.put(deferred)
        return None
    g = run()
    if g is None:
        if hasattr(weight, "grad_added_to_main_grad"):
            weight.grad_added_to_main_grad = True
            weight.grad_added_to_main_grad_once = True
            return torch.zeros(1, dtype=weight.dtype, device=weight.device).expand(weight.shape) \
                if getattr(weight, "zero_out_wgrad", False) else \
                torch.empty(1, dtype=weight.dtype, device=weight.device).expand(weight.shape)
        return None
    return g.reshape(weight.shape)


def bias_grad(dy2d: torch.Tensor, dtype) -> torch.Tensor:
    """Column sums of the output gradient (one two-stage reduction kernel on CUDA)."""
    return ops.column_sum(dy2d, dtype)
