"""LayerNorm / RMSNorm forward and backward (+ fused quantized output).

``y = (x - mu) * rsigma * gamma' + beta`` with ``gamma' = gamma + 1`` when
``zero_centered_gamma``; RMSNorm has ``mu = 0`` and no beta.  Statistics are
fp32.  With a quantizer the CUDA path computes the statistics in one kernel and
lets the tile quantizer apply the normalisation while it quantizes, so the
16-bit normalised tensor is never written
(reference: ``common/normalization/*``, ``pytorch/module/layernorm_linear.py``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _ext
from . import quantize as qz

_ws_cache = {}


def _workspace(dev, numel):
    key = (dev, "norm")
    w = _ws_cache.get(key)
    if w is None or w.numel() < numel:
        w = torch.empty(numel, dtype=torch.float32, device=dev)
        _ws_cache[key] = w
    return w


def norm_fwd_ref(x, gamma, beta, eps, zero_centered, layernorm):
    xf = x.float()
    C = x.shape[-1]
    x2 = xf.reshape(-1, C)
    if layernorm:
        mu = x2.mean(-1)
        var = ((x2 - mu[:, None]) ** 2).mean(-1)
    else:
        mu = None
        var = (x2 * x2).mean(-1)
    rs = torch.rsqrt(var + eps)
    g = gamma.float() + (1.0 if zero_centered else 0.0)
    y = ((x2 - mu[:, None]) if layernorm else x2) * rs[:, None] * g
    if layernorm and beta is not None:
        y = y + beta.float()
    return y.reshape(x.shape), mu, rs


def norm_fwd(x, gamma, beta, eps: float, zero_centered: bool = False, layernorm: bool = False, quantizer=None,
             want_hp: bool = True):
    """Returns (y or None, y_quantized or None, mu or None, rsigma)."""
    C = x.shape[-1]
    R = x.numel() // C
    if _ext.use_cuda(x) and C % 8 == 0 and x.dtype in (torch.bfloat16, torch.float16, torch.float32) \
            and (gamma.dtype == x.dtype or gamma.dtype == torch.float32):
        C_ = _ext.get()
        x = x.contiguous()
        rs = torch.empty(R, dtype=torch.float32, device=x.device)
        mu = torch.empty(R, dtype=torch.float32, device=x.device) if layernorm else None
        yq = None
        fusable = quantizer is not None and _fusable_mx(quantizer, R, C)
        y = torch.empty_like(x) if (want_hp or not fusable) else None
        C_.norm_fwd(layernorm, x, gamma, beta if layernorm else None, y, mu, rs, eps, zero_centered)
        if quantizer is not None:
            if fusable:
                r = qz.fused_quantize_cuda(qz.MODE_MX, x.reshape(R, C), R, C, fp8_dtype=quantizer.dtype,
                                           rowwise=quantizer.rowwise_usage, columnwise=quantizer.columnwise_usage,
                                           prologue=qz.PRO_NORM, mu=mu, rs=rs, gamma=gamma,
                                           beta=beta if layernorm else None, zero_centered=zero_centered)
                yq = quantizer._wrap(r["row_data"].reshape(x.shape) if r["row_data"] is not None else None,
                                     r["row_scale"], r["col_data"], r["col_scale"], tuple(x.shape), x.dtype)
            else:
                yq = quantizer(y)
        return y, yq, mu, rs
    y, mu, rs = norm_fwd_ref(x, gamma, beta, eps, zero_centered, layernorm)
    y = y.to(x.dtype)
    yq = quantizer(y) if quantizer is not None else None
    return y, yq, mu, rs


def _fusable_mx(quantizer, R, C) -> bool:
    from ..tensor.mxfp8 import MXFP8Quantizer

    return isinstance(quantizer, MXFP8Quantizer) and R % 32 == 0 and C % 32 == 0


def norm_bwd_ref(dy, x, mu, rs, gamma, zero_centered, layernorm):
    C = x.shape[-1]
    x2, d2 = x.float().reshape(-1, C), dy.float().reshape(-1, C)
    g = gamma.float() + (1.0 if zero_centered else 0.0)
    xh = ((x2 - mu[:, None]) if layernorm else x2) * rs[:, None]
    dg = d2 * g
    s1 = (dg * xh).mean(-1, keepdim=True)
    dx = dg - xh * s1
    if layernorm:
        dx = dx - dg.mean(-1, keepdim=True)
    dx = dx * rs[:, None]
    dgamma = (d2 * xh).sum(0)
    dbeta = d2.sum(0) if layernorm else None
    return dx.reshape(x.shape), dgamma, dbeta


def norm_bwd(dy, x, mu, rs, gamma, zero_centered: bool = False, layernorm: bool = False,
             add: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Returns (dx [+ add], dgamma, dbeta)."""
    C = x.shape[-1]
    R = x.numel() // C
    if _ext.use_cuda(x) and C % 8 == 0 and x.dtype in (torch.bfloat16, torch.float16, torch.float32) \
            and (gamma.dtype == x.dtype or gamma.dtype == torch.float32):
        C_ = _ext.get()
        dy = dy.contiguous().to(x.dtype)
        x = x.contiguous()
        dx = torch.empty_like(x)
        dgamma = torch.empty_like(gamma)
        dbeta = torch.empty_like(gamma) if layernorm else None
        ws = _workspace(x.device, C_.norm_bwd_workspace(R, C))
        C_.norm_bwd(layernorm, dy, x, mu, rs, gamma, add.contiguous() if add is not None else None, dx, dgamma, dbeta,
                    ws, zero_centered)
        return dx, dgamma, dbeta
    dx, dgamma, dbeta = norm_bwd_ref(dy, x, mu, rs, gamma, zero_centered, layernorm)
    if add is not None:
        dx = dx + add.float()
    return dx.to(x.dtype), dgamma.to(gamma.dtype), dbeta.to(gamma.dtype) if dbeta is not None else None
