"""Quantize / dequantize entry points.

CUDA tensors go to the sm_100a kernels (``csrc/quant``); CPU tensors run the
pure-PyTorch reference math in :mod:`.ref.quant`, which is also the oracle the
kernels are tested against.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import _ext
from .ref import quant as Q

# enums mirrored from csrc/include/teb200/quant.h
PRO_IDENTITY, PRO_NORM, PRO_ACT, PRO_GATED, PRO_DACT, PRO_DGATED = range(6)
MODE_MX, MODE_TENSOR, MODE_NONE = range(3)
ACT_IDS = {"gelu": 0, "silu": 1, "relu": 2, "qgelu": 3, "srelu": 4, "identity": 5}
GATED_ACTS = {"geglu": "gelu", "swiglu": "silu", "reglu": "relu", "qgeglu": "qgelu", "sreglu": "srelu", "glu": "sigmoid"}


def _is_e5m2(dtype: torch.dtype) -> bool:
    return dtype == torch.float8_e5m2


def amax(x: torch.Tensor) -> torch.Tensor:
    """max(|x|) as an fp32 tensor of one element."""
    if _ext.use_cuda(x):
        out = torch.empty(1, dtype=torch.float32, device=x.device)
        _ext.get().amax(x.contiguous(), out)
        return out
    return Q.amax_abs(x)


def mx_scale_numel(rows: int, blocks: int) -> int:
    return Q.round_up(rows, 128) * Q.round_up(blocks, 4)


def fused_quantize_cuda(
    mode: int,
    x: torch.Tensor,
    R: int,
    C: int,
    *,
    fp8_dtype: torch.dtype = torch.float8_e4m3fn,
    rowwise: bool = True,
    columnwise: bool = True,
    prologue: int = PRO_IDENTITY,
    act: str = "gelu",
    dy: Optional[torch.Tensor] = None,
    want_y: bool = False,
    y_dtype: Optional[torch.dtype] = None,
    mu=None,
    rs=None,
    gamma=None,
    beta=None,
    zero_centered: bool = False,
    row_mul=None,
    scale=None,
    amax_out=None,
    dbias: bool = False,
):
    """Run the tile quantizer.  Returns a dict with the produced tensors."""
    C_ = _ext.get()
    dev = x.device
    out = {}
    y = torch.empty(R, C, dtype=y_dtype or x.dtype, device=dev) if want_y else None
    rd = rs_ = cd = cs_ = scale_inv = None
    if mode != MODE_NONE:
        if rowwise:
            rd = torch.empty(R, C, dtype=torch.uint8, device=dev)
        if columnwise:
            cd = torch.empty(C, R, dtype=torch.uint8, device=dev)
        if mode == MODE_MX:
            # padded regions of the scale buffers must be finite: the GEMM reads whole 128x4 tiles
            if rowwise:
                n = mx_scale_numel(R, C // 32)
                rs_ = (torch.zeros if (R % 128 or (C // 32) % 4) else torch.empty)(n, dtype=torch.uint8, device=dev)
            if columnwise:
                n = mx_scale_numel(C, R // 32)
                cs_ = (torch.zeros if (C % 128 or (R // 32) % 4) else torch.empty)(n, dtype=torch.uint8, device=dev)
        else:
            scale_inv = torch.empty(1, dtype=torch.float32, device=dev)
    db = torch.zeros(C, dtype=torch.float32, device=dev) if dbias else None
    C_.quantize(mode, prologue, ACT_IDS.get(act, 0), x, dy, R, C, y, rd, rs_, cd, cs_, _is_e5m2(fp8_dtype), mu, rs,
                gamma, beta, zero_centered, row_mul, scale, amax_out, scale_inv, db)
    out.update(y=y, row_data=rd, row_scale=rs_, col_data=cd, col_scale=cs_, scale_inv=scale_inv, dbias=db)
    return out


# ----------------------------------------------------------------------------- per-tensor FP8
def quantize_fp8(x2d, scale, fp8_dtype, amax_out=None, rowwise=True, columnwise=True):
    """Per-tensor scaled cast.  Returns (data uint8 [R,C] | None, transpose uint8 [C,R] | None, scale_inv)."""
    R, C = x2d.shape
    if _ext.use_cuda(x2d) and R % 32 == 0 and C % 32 == 0 and x2d.dtype in (torch.bfloat16, torch.float16, torch.float32):
        x2d = x2d.contiguous()
        am = amax_out.reshape(-1)[:1] if amax_out is not None else None
        if am is not None and not am.is_contiguous():
            am = None
        r = fused_quantize_cuda(MODE_TENSOR, x2d, R, C, fp8_dtype=fp8_dtype, rowwise=rowwise, columnwise=columnwise,
                                scale=scale.reshape(1).float(), amax_out=am)
        if amax_out is not None and am is None:
            amax_out.copy_(torch.maximum(amax_out.reshape(1), amax(x2d)).reshape(amax_out.shape))
        return r["row_data"], r["col_data"], r["scale_inv"]
    if amax_out is not None:
        amax_out.copy_(torch.maximum(amax_out.reshape(1).float(), Q.amax_abs(x2d).to(amax_out.device)).reshape(amax_out.shape))
    q = Q.quantize_fp8_tensor(x2d, scale.reshape(1), fp8_dtype)
    data = q.view(torch.uint8) if rowwise else None
    tr = q.t().contiguous().view(torch.uint8) if columnwise else None
    return data, tr, (1.0 / scale.reshape(1).float())


def dequantize_fp8(data_u8, scale_inv, fp8_dtype, out_dtype):
    if _ext.use_cuda(data_u8):
        out = torch.empty(data_u8.shape, dtype=out_dtype, device=data_u8.device)
        _ext.get().dequantize_fp8(data_u8.contiguous(), scale_inv.reshape(1).float(), _is_e5m2(fp8_dtype), out)
        return out
    return Q.dequantize_fp8_tensor(data_u8.view(fp8_dtype), scale_inv.reshape(1), out_dtype)


# ----------------------------------------------------------------------------- MXFP8
def quantize_mxfp8(x2d, fp8_dtype, rowwise=True, columnwise=True, two_d: bool = False):
    """Returns (row_data u8 [R,C], row_scales swizzled, col_data_t u8 [C,R], col_scales swizzled).
    ``two_d``: one scale per 32 x 32 block (weights; tensor operations on any device, used once per weight
    update), else per 1 x 32 block along each direction (the fused kernel on a GPU)."""
    R, C = x2d.shape
    if two_d:
        xr = x2d.to(torch.bfloat16).float()
        rd, rs, cd, cs = Q.quantize_mxfp8_2d(xr, fp8_dtype, rowwise, columnwise)
        return (rd.view(torch.uint8) if rd is not None else None, Q.swizzle_scales(rs) if rs is not None else None,
                cd.view(torch.uint8) if cd is not None else None, Q.swizzle_scales(cs) if cs is not None else None)
    if _ext.use_cuda(x2d):
        if x2d.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            x2d = x2d.float()
        r = fused_quantize_cuda(MODE_MX, x2d.contiguous(), R, C, fp8_dtype=fp8_dtype, rowwise=rowwise,
                                columnwise=columnwise)
        return r["row_data"], r["row_scale"], r["col_data"], r["col_scale"]
    # the kernels round through bf16 first; mirror that so both paths agree bit for bit
    xr = x2d.to(torch.bfloat16).float()
    rd, rs, cd, cs = Q.quantize_mxfp8(xr, fp8_dtype, rowwise, columnwise)
    return (
        rd.view(torch.uint8) if rd is not None else None,
        Q.swizzle_scales(rs) if rs is not None else None,
        cd.view(torch.uint8) if cd is not None else None,
        Q.swizzle_scales(cs) if cs is not None else None,
    )


def dequantize_mxfp8(data_u8_2d, scales_swizzled, fp8_dtype, out_dtype):
    R, C = data_u8_2d.shape
    if _ext.use_cuda(data_u8_2d):
        out = torch.empty(R, C, dtype=out_dtype, device=data_u8_2d.device)
        _ext.get().dequantize_mxfp8(data_u8_2d.contiguous(), scales_swizzled, R, C, _is_e5m2(fp8_dtype), out)
        return out
    e = Q.unswizzle_scales(scales_swizzled, R, C // 32)
    return Q.dequantize_mxfp8_rowwise(data_u8_2d.view(fp8_dtype), e, out_dtype)


def swizzle_scales(compact: torch.Tensor) -> torch.Tensor:
    if _ext.use_cuda(compact):
        R, K = compact.shape
        out = torch.zeros(mx_scale_numel(R, K), dtype=torch.uint8, device=compact.device)
        _ext.get().swizzle(compact.contiguous(), R, K, out, True)
        return out
    return Q.swizzle_scales(compact)


def unswizzle_scales(swz: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    if _ext.use_cuda(swz):
        out = torch.empty(rows, cols, dtype=torch.uint8, device=swz.device)
        _ext.get().swizzle(swz, rows, cols, out, False)
        return out
    return Q.unswizzle_scales(swz, rows, cols)


# ----------------------------------------------------------------------------- NVFP4
def quantize_nvfp4(x2d, *, rowwise=True, columnwise=True, with_rht=False, with_2d=False, stochastic_rounding=False,
                   amax_reduce: Optional[Callable] = None, generator=None, four_over_six: Optional[str] = None,
                   e4m3_max: float = 448.0):
    """Returns (row_data [R,C/2], row_scale swz, amax_row, col_data_t [C,R/2], col_scale swz, amax_col).

    ``four_over_six`` (``"MAE"`` / ``"MSE"``): adaptive block scaling, every block keeps the better of the
    map-to-6 and map-to-4 quantizations (``ref/quant.py``); it runs as tensor operations on any device (no fused
    kernel: meant for post-training / RL weights and activations, not for the pre-training hot path) and excludes
    the Hadamard transform and stochastic rounding.  ``e4m3_max`` bounds the block scales (256 leaves room for the
    1.5 x larger map-to-4 scale); it is folded into the returned amax (``amax * 448 / e4m3_max``), so the decode
    side, which derives the tensor scale from that amax, needs no change."""
    R, C = x2d.shape
    reduce = amax_reduce or (lambda a: a)
    if four_over_six and (with_rht or stochastic_rounding):
        raise NotImplementedError("4-over-6 NVFP4 scaling does not combine with the Hadamard transform or "
                                  "stochastic rounding")
    if _ext.use_cuda(x2d) and hasattr(_ext.get(), "quantize_nvfp4") and not four_over_six and e4m3_max == 448.0:
        return _quantize_nvfp4_cuda(x2d, rowwise, columnwise, with_rht, with_2d, stochastic_rounding, reduce)
    xr = x2d.to(torch.bfloat16).float() if x2d.dtype == torch.float32 else x2d.float()
    widen = 448.0 / float(e4m3_max)
    rd = rs = ar = cd = cs = ac = None
    if rowwise:
        ar = reduce(Q.amax_abs(xr)) * widen
        if with_2d:
            d, s = Q.quantize_nvfp4_2d(xr, ar, four_over_six)
        else:
            d, s = Q.quantize_nvfp4_1d(xr, ar, stochastic_rounding, generator, four_over_six)
        rd, rs = d, Q.swizzle_scales(s)
    if columnwise:
        xt = xr.t().contiguous()
        if with_rht:
            xt = Q.apply_rht(xt)
        ac = reduce(Q.amax_abs(xt)) * widen
        if with_2d:
            d, s = Q.quantize_nvfp4_2d(xt, ac, four_over_six)
        else:
            d, s = Q.quantize_nvfp4_1d(xt, ac, stochastic_rounding, generator, four_over_six)
        cd, cs = d, Q.swizzle_scales(s)
    return rd, rs, ar, cd, cs, ac


def _quantize_nvfp4_cuda(x2d, rowwise, columnwise, with_rht, with_2d, sr, reduce):
    C_ = _ext.get()
    R, C = x2d.shape
    dev = x2d.device
    x2d = x2d.contiguous()
    if x2d.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        x2d = x2d.float()
    am = torch.zeros(2, dtype=torch.float32, device=dev)
    C_.nvfp4_amax(x2d, R, C, bool(with_rht and columnwise), am)
    ar = reduce(am[0:1].clone()) if rowwise else None
    ac = reduce(am[1:2].clone() if with_rht else am[0:1].clone()) if columnwise else None
    rd = torch.empty(R, C // 2, dtype=torch.uint8, device=dev) if rowwise else None
    rs = torch.zeros(mx_scale_numel(R, C // 16), dtype=torch.uint8, device=dev) if rowwise else None
    cd = torch.empty(C, R // 2, dtype=torch.uint8, device=dev) if columnwise else None
    cs = torch.zeros(mx_scale_numel(C, R // 16), dtype=torch.uint8, device=dev) if columnwise else None
    seed, ctr = 0, None
    if sr:
        # the stream of random numbers is (seed, call counter): the counter lives on the device and is advanced
        # by a device op, so there is no host synchronisation and a captured graph draws new numbers per replay
        seed = int(torch.cuda.initial_seed())
        ctr = _SR_COUNTERS.get(dev)
        if ctr is None:
            ctr = _SR_COUNTERS[dev] = torch.zeros(1, dtype=torch.int64, device=dev)
        ctr.add_(0x9E3779B1)
    C_.quantize_nvfp4(x2d, R, C, ar, ac, rd, rs, cd, cs, bool(with_rht), bool(with_2d), bool(sr), seed, 0, ctr)
    return rd, rs, ar, cd, cs, ac


_SR_COUNTERS: dict = {}


def dequantize_nvfp4(packed, scales_swizzled, amax_t, R, C, out_dtype):
    if _ext.use_cuda(packed) and hasattr(_ext.get(), "dequantize_nvfp4"):
        out = torch.empty(R, C, dtype=out_dtype, device=packed.device)
        _ext.get().dequantize_nvfp4(packed.contiguous(), scales_swizzled, amax_t, R, C, out)
        return out
    s = Q.unswizzle_scales(scales_swizzled, R, C // 16)
    return Q.dequantize_nvfp4(packed.reshape(R, C // 2), s, amax_t, out_dtype)


def hadamard_transform(x2d: torch.Tensor, transposed: bool = False) -> torch.Tensor:
    """The 16-point randomised Hadamard transform that the NVFP4 quantizer applies, as a stand-alone operation:
    every block of 16 consecutive values of a row is multiplied by ``diag(signs) H16 / 4`` (an orthogonal matrix,
    fixed sign vector).  ``transposed=True`` rotates the rows of ``x^T`` (blocks of 16 consecutive ROWS of ``x``, the
    token dimension of a weight-gradient operand) and returns ``[C, R]``.  Inside the quantizer the rotation is fused
    with the cast; this form exists for analysis and tests.  (Reference: ``common/hadamard_transform/hadamard_transform.cu:328``.)"""
    x = x2d.t().contiguous() if transposed else x2d
    assert x.dim() == 2 and x.shape[1] % 16 == 0, "the rotated dimension must be a multiple of 16"
    return Q.apply_rht(x)
