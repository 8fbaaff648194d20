"""Front end of the library's own fused attention kernels (``csrc/attn``): tcgen05 forward,
dK/dV and dQ kernels for head dim 128 in fp16/bf16 with causal masks and grouped-query heads.

All tensors are ``[b, h, s, d]`` VIEWS; the kernels read them through 4-D TMA descriptors, so
``sbhd``/``bshd`` projections are consumed without a copy.  (Reference counterpart:
``pytorch/cpp_extensions/fused_attn.py:127, 386`` over cuDNN.)
"""
from __future__ import annotations

import torch

from . import _ext


def _view_ok(t: torch.Tensor) -> bool:
    return t.dim() == 4 and t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3])


def supported(q, k, v, causal) -> bool:
    if not _ext.available() or not hasattr(_ext.get(), "flash_fwd"):
        return False
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        return False
    if q.shape[-1] != 128 or k.shape[-1] != 128 or v.shape[-1] != 128 or q.shape[1] % k.shape[1] != 0:
        return False
    if k.shape[2] != v.shape[2] or k.shape[1] != v.shape[1] or q.shape[2] == 0 or k.shape[2] == 0:
        return False
    return all(t.stride(3) == 1 or t.is_contiguous() for t in (q, k, v))


def _prep(t: torch.Tensor) -> torch.Tensor:
    return t if _view_ok(t) else t.contiguous()


def _empty_out(q: torch.Tensor, out_format: str) -> torch.Tensor:
    b, h, s, d = q.shape
    if out_format == "sbhd":
        return torch.empty(s, b, h, d, dtype=q.dtype, device=q.device).permute(1, 2, 0, 3)
    if out_format == "bshd":
        return torch.empty(b, s, h, d, dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    return torch.empty(b, h, s, d, dtype=q.dtype, device=q.device)


class _FlashFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, bottom_right, out_format):  # type: ignore[override]
        C_ = _ext.get()
        q, k, v = _prep(q), _prep(k), _prep(v)
        b, h, sq, d = q.shape
        out = _empty_out(q, out_format)
        s_pad = (sq + 127) // 128 * 128  # the backward reads lse / delta in blocks of 128 rows
        lse = torch.empty(b, h, s_pad, dtype=torch.float32, device=q.device)
        sc = float(scale) if scale is not None else d ** -0.5
        C_.flash_fwd(q, k, v, out, lse, sc, bool(causal), bool(bottom_right), C_.status(q.device.index))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (sc, bool(causal), bool(bottom_right))
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        C_ = _ext.get()
        q, k, v, out, lse = ctx.saved_tensors
        sc, causal, bottom_right = ctx.cfg
        dout = _prep(dout)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if dk.stride() != dv.stride():
            dv = torch.empty_strided(dk.shape, dk.stride(), dtype=dk.dtype, device=dk.device)
        delta = torch.empty_like(lse)
        C_.flash_bwd(dout, q, k, v, out, lse, delta, dq, dk, dv, sc, causal, bottom_right,
                     C_.status(q.device.index))
        return dq, dk, dv, None, None, None, None


def flash_attention(q, k, v, scale, causal, bottom_right=True, out_format: str = "bhsd"):
    return _FlashFunc.apply(q, k, v, scale, causal, bottom_right, out_format)


def flash_forward_lse(q, k, v, scale, causal, bottom_right=True):
    """Forward only, returning (out, lse[b, h, sq]) for merging partial results (context parallel)."""
    C_ = _ext.get()
    q, k, v = _prep(q), _prep(k), _prep(v)
    b, h, sq, d = q.shape
    out = _empty_out(q, "bhsd")
    s_pad = (sq + 127) // 128 * 128  # the backward reads lse / delta in blocks of 128 rows
    lse = torch.empty(b, h, s_pad, dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else d ** -0.5
    C_.flash_fwd(q, k, v, out, lse, sc, bool(causal), bool(bottom_right), C_.status(q.device.index))
    return out, lse[:, :, :sq]
