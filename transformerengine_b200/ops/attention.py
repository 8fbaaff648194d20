"""Scaled dot-product attention (forward + backward) with causal / padding /
sliding-window masks, GQA, bias, dropout and the softmax variants (vanilla,
off-by-one, learnable sink).

Layouts are ``[b, h, s, d]`` internally.  The reference math runs in fp32 and is
the oracle (reference: ``pytorch/attention/dot_product_attention/backends.py:351``
UnfusedDotProductAttention and the cuDNN graphs of ``common/fused_attn``).
"""
from __future__ import annotations

import os

import math
from typing import Optional, Tuple

import torch

from . import _ext


def _build_mask(sq, sk, device, causal, window, bottom_right=True):
    """True = masked out.  ``window`` = (left, right) with -1 meaning unbounded."""
    if not causal and (window is None or (window[0] < 0 and window[1] < 0)):
        return None
    qi = torch.arange(sq, device=device)[:, None]
    ki = torch.arange(sk, device=device)[None, :]
    off = (sk - sq) if bottom_right else 0
    rel = ki - (qi + off)  # >0: key in the future
    m = torch.zeros(sq, sk, dtype=torch.bool, device=device)
    right = 0 if causal else (window[1] if window is not None else -1)
    left = window[0] if window is not None else -1
    if right >= 0:
        m |= rel > right
    if left >= 0:
        m |= rel < -left
    return m


def attention_ref(q, k, v, *, scale=None, causal=False, window=None, attn_mask=None, bias=None, dropout_p=0.0,
                  softmax_type="vanilla", sink=None, bottom_right=True, generator=None, return_lse=False,
                  score_mod=None, score_mod_tensors=None):
    """fp32 attention on ``[b, h, s, d]`` tensors; k/v may have fewer heads (GQA).
    ``score_mod(score, tensors) -> score`` edits the scaled scores ``[b, h, sq, sk]`` before masking."""
    b, hq, sq, d = q.shape
    hk, sk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qf, kf, vf = q.float(), k.float(), v.float()
    if hk != hq:
        rep = hq // hk
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if bias is not None:
        s = s + bias.float()
    if score_mod is not None:
        s = score_mod(s, score_mod_tensors or {})
    m = _build_mask(sq, sk, q.device, causal, window, bottom_right)
    if m is not None:
        s = s.masked_fill(m, float("-inf"))
    if attn_mask is not None:
        s = s.masked_fill(attn_mask, float("-inf"))
    if softmax_type == "vanilla":
        lse = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - lse[..., None])
    else:
        # one extra logit per row: 0 (off-by-one) or a learnable per-head sink
        extra = torch.zeros(b, hq, sq, 1, device=q.device) if softmax_type == "off-by-one" else \
            sink.float().reshape(1, hq, 1, 1).expand(b, hq, sq, 1)
        lse = torch.logsumexp(torch.cat([s, extra], dim=-1), dim=-1)
        p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    if dropout_p > 0.0:
        keep = torch.rand(p.shape, device=p.device, generator=generator) >= dropout_p
        p = p * keep / (1 - dropout_p)
    o = torch.matmul(p, vf).to(q.dtype)
    return (o, lse) if return_lse else o


@torch.no_grad()
def max_attention_logit(q, k, *, scale=None, causal=False, window=None, attn_mask=None, bias=None,
                        bottom_right=True, chunk_bytes: int = 256 << 20) -> torch.Tensor:
    """Per-head maximum of the scaled, biased and masked attention scores of ``[b, h, s, d]`` tensors (fp32 ``[h]``;
    the quantity "QK-clip" optimizers watch).  A pass of its own over Q K^T in blocks of query rows, so that no
    ``s x s`` score tensor is kept.  (Reference: ``return_max_logit`` of
    ``attention/dot_product_attention/backends.py``.)"""
    b, hq, sq, d = q.shape
    hk, sk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    kf = k.float()
    if hk != hq:
        kf = kf.repeat_interleave(hq // hk, dim=1)
    kt = kf.transpose(-1, -2)
    m = _build_mask(sq, sk, q.device, causal, window, bottom_right)
    rows = max(1, min(sq, chunk_bytes // max(4 * b * hq * sk, 1)))
    best = torch.full((hq,), float("-inf"), dtype=torch.float32, device=q.device)
    for r0 in range(0, sq, rows):
        r1 = min(r0 + rows, sq)
        s = torch.matmul(q[:, :, r0:r1].float(), kt) * scale
        if bias is not None:
            bb = bias.float()
            s = s + (bb[..., r0:r1, :] if bb.shape[-2] == sq else bb)
        if m is not None:
            s = s.masked_fill(m[r0:r1], float("-inf"))
        if attn_mask is not None:
            am = attn_mask
            s = s.masked_fill(am[..., r0:r1, :] if am.shape[-2] == sq else am, float("-inf"))
        best = torch.maximum(best, s.amax(dim=(0, 2, 3)))
    return best


_USE_LIBRARY_SDPA = True
# attention_backend='library' (TEB200_ATTN=library) routes the plain 16-bit case to torch's SDPA instead of
# csrc/attn (A/B timing)
from ..utils.config import get_config as _get_config  # noqa: E402

_USE_OWN_FLASH = _get_config().attention_backend == "own"
_USE_LIBRARY_SDPA = _get_config().attention_backend != "reference"


def attention(q, k, v, *, scale=None, causal=False, window=None, attn_mask=None, bias=None, dropout_p=0.0,
              softmax_type="vanilla", sink=None, bottom_right=True, out_format="bhsd", score_mod=None,
              score_mod_tensors=None):
    """Differentiable attention on ``[b, h, s, d]``; ``out_format`` names the memory layout of the
    returned ``[b, h, s, d]`` view ("bhsd", "sbhd" or "bshd") when the fused kernel runs.

    On CUDA the fused flash kernel of this library handles the common case
    (16-bit, no bias / arbitrary mask / dropout, head dim 64 or 128); everything
    else runs the reference math, which autograd differentiates.
    """
    no_window = window is None or (window[0] < 0 and (window[1] < 0 or (causal and window[1] == 0)))
    plain = attn_mask is None and bias is None and dropout_p == 0.0 and softmax_type == "vanilla" and \
        score_mod is None
    if _ext.use_cuda(q) and plain and q.dtype in (torch.bfloat16, torch.float16):
        from . import flash

        if _USE_OWN_FLASH and flash.supported(q, k, v, causal):
            return flash.flash_attention(q, k, v, scale, causal, bottom_right, out_format,
                                         None if no_window else window)
        if _USE_LIBRARY_SDPA and no_window and (not causal or q.shape[2] == k.shape[2] or not bottom_right):
            return torch.nn.functional.scaled_dot_product_attention(
                q, k, v, is_causal=causal, scale=scale, enable_gqa=q.shape[1] != k.shape[1])
    return attention_ref(q, k, v, scale=scale, causal=causal, window=window, attn_mask=attn_mask, bias=bias,
                         dropout_p=dropout_p, softmax_type=softmax_type, sink=sink, bottom_right=bottom_right,
                         score_mod=score_mod, score_mod_tensors=score_mod_tensors)


def merge_attention_states(o1, lse1, o2, lse2) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combine two partial attention results over disjoint key sets (ring / context parallel)."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse)[..., None]
    w2 = torch.exp(lse2 - lse)[..., None]
    w1 = torch.nan_to_num(w1, nan=0.0)
    w2 = torch.nan_to_num(w2, nan=0.0)
    return (o1.float() * w1 + o2.float() * w2).to(o1.dtype), lse
