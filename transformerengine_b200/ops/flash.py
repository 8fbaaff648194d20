"""Front end of the library's own fused attention kernels (``csrc/attn``)."""
from __future__ import annotations

import torch

from . import _ext


def supported(q, k, v, causal) -> bool:
    if not _ext.available():
        return False
    C_ = _ext.get()
    if not hasattr(C_, "flash_fwd"):
        return False
    d = q.shape[-1]
    return d in (64, 128) and q.shape[2] % 128 == 0 and k.shape[2] % 128 == 0 and q.shape[1] % k.shape[1] == 0 \
        and v.shape[-1] == d


class _FlashFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, bottom_right):  # type: ignore[override]
        C_ = _ext.get()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        b, h, sq, d = q.shape
        out = torch.empty_like(q)
        lse = torch.empty(b, h, sq, dtype=torch.float32, device=q.device)
        sc = scale if scale is not None else d ** -0.5
        C_.flash_fwd(q, k, v, out, lse, float(sc), bool(causal))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.sc, ctx.causal = sc, causal
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        C_ = _ext.get()
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        C_.flash_bwd(dout.contiguous(), q, k, v, out, lse, dq, dk, dv, float(ctx.sc), bool(ctx.causal))
        return dq, dk, dv, None, None, None


def flash_attention(q, k, v, scale, causal, bottom_right=True):
    return _FlashFunc.apply(q, k, v, scale, causal, bottom_right)
