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
    def forward(ctx, q, k, v, scale, causal, bottom_right, out_format, window):  # type: ignore[override]
        C_ = _ext.get()
        q, k, v = _prep(q), _prep(k), _prep(v)
        b, h, sq, d = q.shape
        out = _empty_out(q, out_format)
        s_pad = (sq + 127) // 128 * 128  # the backward reads lse / delta in blocks of 128 rows
        lse = torch.empty(b, h, s_pad, dtype=torch.float32, device=q.device)
        sc = float(scale) if scale is not None else d ** -0.5
        wl, wr = (-1, -1) if window is None else (int(window[0]), int(window[1]))
        C_.flash_fwd(q, k, v, out, lse, sc, bool(causal), bool(bottom_right), C_.status(q.device.index),
                     window_left=wl, window_right=wr)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (sc, bool(causal), bool(bottom_right), wl, wr)
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        C_ = _ext.get()
        q, k, v, out, lse = ctx.saved_tensors
        sc, causal, bottom_right, wl, wr = ctx.cfg
        dout = _prep(dout)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if dk.stride() != dv.stride():
            dv = torch.empty_strided(dk.shape, dk.stride(), dtype=dk.dtype, device=dk.device)
        delta = torch.empty_like(lse)
        C_.flash_bwd(dout, q, k, v, out, lse, delta, dq, dk, dv, sc, causal, bottom_right,
                     C_.status(q.device.index), window_left=wl, window_right=wr)
        return dq, dk, dv, None, None, None, None, None


def flash_attention(q, k, v, scale, causal, bottom_right=True, out_format: str = "bhsd", window=None):
    """``window = (left, right)``: query i sees keys [i - left, i + right] around the (bottom-right or
    top-left aligned) diagonal, -1 = unbounded; ``causal`` forces right = 0."""
    if window is not None and window[0] < 0 and window[1] < 0:
        window = None
    return _FlashFunc.apply(q, k, v, scale, causal, bottom_right, out_format, window)


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


# ---------------------------------------------------------------------------------------------
# Packed variable-length sequences ("thd"): the kernels take the cumulative lengths and walk every
# sequence inside one launch (reference: cu_seqlens / cu_seqlens_padded arguments of
# ``pytorch/cpp_extensions/fused_attn.py:127``).
def supported_varlen(q, k, v) -> bool:
    if not _ext.available() or not hasattr(_ext.get(), "flash_fwd_varlen"):
        return False
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3 or k.shape != v.shape:
        return False
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        return False
    return q.shape[-1] == 128 and k.shape[-1] == 128 and q.shape[1] % k.shape[1] == 0 and q.shape[0] > 0 and k.shape[0] > 0


def _thd_view(t: torch.Tensor) -> torch.Tensor:
    """[t, h, d] -> [1, h, t, d] view (copy only if the layout cannot be described to TMA)."""
    v = t.permute(1, 0, 2).unsqueeze(0)
    return v if _view_ok(v) else t.contiguous().permute(1, 0, 2).unsqueeze(0)


class _FlashVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, off_q, off_k, max_sq, max_sk, scale, causal, bottom_right, window):  # type: ignore[override]
        C_ = _ext.get()
        tq, hq, d = q.shape
        nseq = cu_q.numel() - 1
        out = torch.zeros(tq, hq, d, dtype=q.dtype, device=q.device)  # tokens outside every sequence stay 0
        s_pad = (max_sq + 127) // 128 * 128
        lse = torch.empty(nseq, hq, s_pad, dtype=torch.float32, device=q.device)
        sc = float(scale) if scale is not None else d ** -0.5
        qv, kv, vv = _thd_view(q), _thd_view(k), _thd_view(v)
        wl, wr = (-1, -1) if window is None else (int(window[0]), int(window[1]))
        C_.flash_fwd_varlen(qv, kv, vv, _thd_view(out), lse, cu_q, cu_k, off_q, off_k, max_sq, max_sk, sc,
                            bool(causal), bool(bottom_right), C_.status(q.device.index), window_left=wl,
                            window_right=wr)
        ctx.save_for_backward(qv, kv, vv, out, lse, cu_q, cu_k, off_q, off_k)
        ctx.cfg = (sc, bool(causal), bool(bottom_right), max_sq, max_sk, wl, wr)
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        C_ = _ext.get()
        qv, kv, vv, out, lse, cu_q, cu_k, off_q, off_k = ctx.saved_tensors
        sc, causal, bottom_right, max_sq, max_sk, wl, wr = ctx.cfg
        dq = torch.zeros(qv.shape[2], qv.shape[1], 128, dtype=qv.dtype, device=qv.device)
        dk = torch.zeros(kv.shape[2], kv.shape[1], 128, dtype=qv.dtype, device=qv.device)
        dv = torch.zeros_like(dk)
        delta = torch.empty_like(lse)
        C_.flash_bwd_varlen(_thd_view(dout), qv, kv, vv, _thd_view(out), lse, delta, _thd_view(dq), _thd_view(dk),
                            _thd_view(dv), cu_q, cu_k, off_q, off_k, max_sq, max_sk, sc, causal, bottom_right,
                            C_.status(qv.device.index), window_left=wl, window_right=wr)
        return (dq, dk, dv) + (None,) * 10


def flash_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_kv, scale=None, causal=False, bottom_right=True,
                           max_seqlen_q=None, max_seqlen_kv=None, cu_seqlens_q_padded=None,
                           cu_seqlens_kv_padded=None, window=None):
    """Attention over packed sequences.  ``q`` is ``[tq, hq, 128]``, ``k`` / ``v`` ``[tk, hk, 128]``;
    sequence i owns ``cu_seqlens[i+1] - cu_seqlens[i]`` tokens starting at ``cu_seqlens_padded[i]``
    (``cu_seqlens[i]`` when no padded offsets are given).  Returns ``[tq, hq, 128]``."""
    cu_q = cu_seqlens_q.to(device=q.device, dtype=torch.int32).contiguous()
    cu_k = cu_seqlens_kv.to(device=q.device, dtype=torch.int32).contiguous()
    off_q = cu_q if cu_seqlens_q_padded is None else cu_seqlens_q_padded.to(device=q.device, dtype=torch.int32).contiguous()
    off_k = cu_k if cu_seqlens_kv_padded is None else cu_seqlens_kv_padded.to(device=q.device, dtype=torch.int32).contiguous()
    if max_seqlen_q is None:
        max_seqlen_q = int((cu_q[1:] - cu_q[:-1]).max())
    if max_seqlen_kv is None:
        max_seqlen_kv = int((cu_k[1:] - cu_k[:-1]).max())
    if max_seqlen_q <= 0 or max_seqlen_kv <= 0:
        return torch.zeros_like(q)
    if window is not None and window[0] < 0 and (window[1] < 0 or (causal and window[1] == 0)):
        window = None
    return _FlashVarlenFunc.apply(q, k, v, cu_q, cu_k, off_q, off_k, int(max_seqlen_q), int(max_seqlen_kv), scale,
                                  causal, bottom_right, window)
