"""Activation functions, forward and backward, with optional fused quantization.

All math is fp32.  ``gelu`` is the tanh approximation; gated variants read an
input row ``[2n]`` whose first half feeds the activation and whose second half
is the linear multiplier (reference: ``common/util/math.h:20-156``,
``common/util/vectorized_pointwise.h:410-470``).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _ext
from . import quantize as qz

GATED = {"geglu": "gelu", "swiglu": "silu", "reglu": "relu", "qgeglu": "qgelu", "sreglu": "srelu"}
PLAIN = ("gelu", "silu", "relu", "qgelu", "srelu")


def is_gated(name: str) -> bool:
    return name in GATED or name in ("glu", "clamped_swiglu")


def _clamped_params(params):
    p = dict(limit=7.0, alpha=1.702, glu_linear_offset=1.0)
    p.update(params or {})
    return float(p["limit"]), float(p["alpha"]), float(p["glu_linear_offset"])


def _clamped_swiglu_fwd(x1, x2, params):
    """GPT-OSS gated unit: gate input capped at ``limit``, sigmoid(alpha x) gate, linear half clamped to
    +-limit and shifted by ``glu_linear_offset`` (reference: ``common/util/math.h``, ``clamped_silu``)."""
    limit, alpha, off = _clamped_params(params)
    a = torch.clamp(x1, max=limit)
    return a * torch.sigmoid(alpha * a) * (torch.clamp(x2, -limit, limit) + off)


def _clamped_swiglu_bwd(df, x1, x2, params):
    limit, alpha, off = _clamped_params(params)
    a = torch.clamp(x1, max=limit)
    s = torch.sigmoid(alpha * a)
    act = a * s
    dact = (s + alpha * a * s * (1 - s)) * (x1 <= limit)
    lin = torch.clamp(x2, -limit, limit) + off
    dlin = ((x2 >= -limit) & (x2 <= limit)).to(df.dtype)
    return torch.cat([df * lin * dact, df * act * dlin], dim=-1)


def _act(x, name):
    if name == "gelu":
        return x * (0.5 + 0.5 * torch.tanh(x * (0.79788456 + 0.03567741 * x * x)))
    if name == "silu":
        return x * torch.sigmoid(x)
    if name == "relu":
        return torch.relu(x)
    if name == "qgelu":
        return x * torch.sigmoid(1.702 * x)
    if name == "srelu":
        return torch.relu(x) ** 2
    if name == "sigmoid":
        return torch.sigmoid(x)
    raise ValueError(name)


def _dact(x, name):
    if name == "gelu":
        t = torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x))
        return 0.5 * x * ((1 - t * t) * (0.79788456 + 0.1070322243 * x * x)) + 0.5 * (1 + t)
    if name == "silu":
        s = torch.sigmoid(x)
        return s * (1 + x * (1 - s))
    if name == "relu":
        return (x > 0).to(x.dtype)
    if name == "qgelu":
        s = torch.sigmoid(1.702 * x)
        return s + 1.702 * x * s * (1 - s)
    if name == "srelu":
        return 2 * torch.relu(x)
    if name == "sigmoid":
        s = torch.sigmoid(x)
        return s * (1 - s)
    raise ValueError(name)


def activation_fwd_ref(x, name, row_scale=None, params=None):
    xf = x.float()
    if name == "clamped_swiglu":
        n = x.shape[-1] // 2
        y = _clamped_swiglu_fwd(xf[..., :n], xf[..., n:], params)
    elif is_gated(name):
        n = x.shape[-1] // 2
        base = GATED.get(name, "sigmoid")
        y = _act(xf[..., :n], base) * xf[..., n:]
    else:
        y = _act(xf, name)
    if row_scale is not None:
        y = y * row_scale.float().reshape(*y.shape[:-1], 1)
    return y


def activation_bwd_ref(dy, x, name, row_scale=None, params=None):
    xf, df = x.float(), dy.float()
    if row_scale is not None:
        df = df * row_scale.float().reshape(*df.shape[:-1], 1)
    if name == "clamped_swiglu":
        n = x.shape[-1] // 2
        return _clamped_swiglu_bwd(df, xf[..., :n], xf[..., n:], params)
    if is_gated(name):
        n = x.shape[-1] // 2
        base = GATED.get(name, "sigmoid")
        x1, x2 = xf[..., :n], xf[..., n:]
        return torch.cat([df * x2 * _dact(x1, base), df * _act(x1, base)], dim=-1)
    return df * _dact(xf, name)


def _cuda_ok(x, name, C_out):
    R = x.numel() // x.shape[-1]
    return (_ext.use_cuda(x) and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and R % 32 == 0
            and C_out % 32 == 0 and (name in PLAIN or name in GATED))


def activation_fwd(x, name: str, quantizer=None, want_hp: bool = True, row_scale: Optional[torch.Tensor] = None,
                   params: Optional[dict] = None):
    """Returns (y or None, y_quantized or None).  ``params``: ``limit`` / ``alpha`` / ``glu_linear_offset`` of
    ``"clamped_swiglu"`` (which, like ``"glu"``, runs as tensor math on every device)."""
    C_in = x.shape[-1]
    C_out = C_in // 2 if is_gated(name) else C_in
    R = x.numel() // C_in
    out_shape = tuple(x.shape[:-1]) + (C_out,)
    if _cuda_ok(x, name, C_out):
        from ..tensor.mxfp8 import MXFP8Quantizer

        x2 = x.contiguous().reshape(R, C_in)
        gated = is_gated(name)
        base = GATED.get(name, name)
        fuse = isinstance(quantizer, MXFP8Quantizer)
        r = qz.fused_quantize_cuda(
            qz.MODE_MX if fuse else qz.MODE_NONE, x2, R, C_out,
            fp8_dtype=quantizer.dtype if fuse else torch.float8_e4m3fn,
            rowwise=quantizer.rowwise_usage if fuse else False,
            columnwise=quantizer.columnwise_usage if fuse else False,
            prologue=qz.PRO_GATED if gated else qz.PRO_ACT, act=base,
            want_y=want_hp or not fuse, y_dtype=x.dtype,
            row_mul=row_scale.float().reshape(-1).contiguous() if row_scale is not None else None)
        y = r["y"].reshape(out_shape) if r["y"] is not None else None
        yq = None
        if fuse:
            yq = quantizer._wrap(r["row_data"].reshape(out_shape) if r["row_data"] is not None else None,
                                 r["row_scale"], r["col_data"], r["col_scale"], out_shape, x.dtype)
        elif quantizer is not None:
            yq = quantizer(y)
        return y, yq
    y = activation_fwd_ref(x, name, row_scale, params).to(x.dtype)
    return y, (quantizer(y) if quantizer is not None else None)


def activation_bwd(dy, x, name: str, quantizer=None, want_hp: bool = True, want_dbias: bool = False,
                   row_scale: Optional[torch.Tensor] = None, params: Optional[dict] = None):
    """Returns (dx or None, dx_quantized or None, dbias or None)."""
    C_in = x.shape[-1]
    R = x.numel() // C_in
    if _cuda_ok(x, name, C_in) and dy.dtype == x.dtype:
        from ..tensor.mxfp8 import MXFP8Quantizer

        gated = is_gated(name)
        base = GATED.get(name, name)
        fuse = isinstance(quantizer, MXFP8Quantizer)
        r = qz.fused_quantize_cuda(
            qz.MODE_MX if fuse else qz.MODE_NONE, x.contiguous().reshape(R, C_in), R, C_in,
            fp8_dtype=quantizer.dtype if fuse else torch.float8_e4m3fn,
            rowwise=quantizer.rowwise_usage if fuse else False,
            columnwise=quantizer.columnwise_usage if fuse else False,
            prologue=qz.PRO_DGATED if gated else qz.PRO_DACT, act=base, dy=dy.contiguous(),
            want_y=want_hp or not fuse, y_dtype=x.dtype, dbias=want_dbias,
            row_mul=row_scale.float().reshape(-1).contiguous() if row_scale is not None else None)
        dx = r["y"].reshape(x.shape) if r["y"] is not None else None
        dq = None
        if fuse:
            dq = quantizer._wrap(r["row_data"].reshape(x.shape) if r["row_data"] is not None else None,
                                 r["row_scale"], r["col_data"], r["col_scale"], tuple(x.shape), x.dtype)
        elif quantizer is not None:
            dq = quantizer(dx)
        return dx, dq, (r["dbias"] if want_dbias else None)
    dx = activation_bwd_ref(dy, x, name, row_scale, params).to(x.dtype)
    db = dx.reshape(-1, C_in).float().sum(0) if want_dbias else None
    return dx, (quantizer(dx) if quantizer is not None else None), db
