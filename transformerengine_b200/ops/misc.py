"""RoPE, cross entropy, softmax, dropout and multi-tensor optimizer ops."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import _ext

MT_CHUNK = 16 * 1024  # elements per chunk; a fixed grid of blocks strides over the chunks of a launch


# ----------------------------------------------------------------------------- RoPE
def rope_freqs(positions: torch.Tensor, dim: int, base: float = 10000.0, interleaved: bool = False) -> torch.Tensor:
    """Angles ``[len, dim]`` = cat(freqs, freqs) (or interleaved repeat), fp32."""
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=positions.device) / dim))
    f = torch.outer(positions.float(), inv)
    if interleaved:
        return torch.stack([f, f], dim=-1).reshape(f.shape[0], -1)
    return torch.cat([f, f], dim=-1)


def _rotate(x, interleaved):
    if interleaved:
        x1, x2 = x[..., 0::2], x[..., 1::2]
        return torch.stack([-x2, x1], dim=-1).reshape(x.shape)
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def _cp_positions(s, cp_size, cp_rank, device):
    idx = torch.arange(s, device=device)
    if cp_size <= 1:
        return idx
    half = s // 2
    return torch.where(idx < half, idx + cp_rank * half, idx + s * cp_size - (cp_rank + 1) * half - half)


def rope_ref(x_sbhd, freqs, d_rot, interleaved=False, backward=False, pos_offset=0, cp_size=1, cp_rank=0,
             start_positions=None):
    s, b = x_sbhd.shape[0], x_sbhd.shape[1]
    pos = _cp_positions(s, cp_size, cp_rank, x_sbhd.device) + pos_offset
    if start_positions is not None:
        pos = pos[:, None] + start_positions[None, :].to(pos.device)  # [s, b]
        f = freqs[pos][:, :, None, :]
    else:
        f = freqs[pos][:, None, None, :]
    xf = x_sbhd.float()
    xr, xp = xf[..., :d_rot], xf[..., d_rot:]
    cos, sin = torch.cos(f), torch.sin(f)
    if not backward:
        yr = xr * cos + _rotate(xr, interleaved) * sin
    else:
        # transpose of the rotation: rot^T(v) = -rot(v)
        yr = xr * cos - _rotate(xr * sin, interleaved)
    return torch.cat([yr, xp], dim=-1).to(x_sbhd.dtype)


def rope_apply(x_sbhd: torch.Tensor, freqs: torch.Tensor, *, interleaved=False, backward=False, pos_offset=0,
               cp_size=1, cp_rank=0, start_positions=None, inplace=False) -> torch.Tensor:
    """Rotary embedding on a ``[s, b, h, d]`` view (strided views are fine on CUDA)."""
    d_rot = freqs.shape[-1]
    if _ext.use_cuda(x_sbhd) and x_sbhd.stride(-1) == 1 and x_sbhd.dtype in (torch.bfloat16, torch.float16, torch.float32):
        out = x_sbhd if inplace else torch.empty_strided(x_sbhd.shape, x_sbhd.stride(), dtype=x_sbhd.dtype,
                                                         device=x_sbhd.device)
        sp = start_positions.to(torch.int32) if start_positions is not None else None
        _ext.get().rope(x_sbhd, out, freqs.float().contiguous(), d_rot, interleaved, backward, pos_offset, cp_size,
                        cp_rank, sp)
        return out
    y = rope_ref(x_sbhd, freqs.float(), d_rot, interleaved, backward, pos_offset, cp_size, cp_rank, start_positions)
    if inplace:
        x_sbhd.copy_(y)
        return x_sbhd
    return y


def rope_qkv(x_sbhd: torch.Tensor, q_freqs: torch.Tensor, k_freqs: torch.Tensor, *, layout: str, hq: int, hk: int,
             interleaved=False, backward=False, cp_size=1, cp_rank=0, start_positions=None, inplace=False) -> torch.Tensor:
    """Rotary embedding of the query and key heads of a packed QKV projection ``[s, b, hq + 2 hk, d]`` in ONE launch;
    value heads pass through.  ``layout``: ``"grouped"`` = per key/value group ``[hq / hk query heads, key, value]``,
    ``"blocked"`` = ``[hq query heads | hk key heads | hk value heads]``.  (Reference: the fused QKV RoPE of
    ``common/fused_rope/fused_rope.cu:505,551``.)"""
    assert layout in ("grouped", "blocked") and x_sbhd.shape[2] == hq + 2 * hk and hq % hk == 0
    d_rot = q_freqs.shape[-1]
    g = hq // hk
    if _ext.use_cuda(x_sbhd) and x_sbhd.stride(-1) == 1 and x_sbhd.dtype in (torch.bfloat16, torch.float16) \
            and d_rot % 16 == 0 and x_sbhd.data_ptr() % 16 == 0 and all(st % 8 == 0 for st in x_sbhd.stride()[:3]):
        out = x_sbhd if inplace else torch.empty_strided(x_sbhd.shape, x_sbhd.stride(), dtype=x_sbhd.dtype,
                                                         device=x_sbhd.device)
        sp = start_positions.to(torch.int32) if start_positions is not None else None
        fq = q_freqs.float().contiguous()
        fk = None if k_freqs is q_freqs else k_freqs.float().contiguous()
        _ext.get().rope(x_sbhd, out, fq, d_rot, interleaved, backward, 0, cp_size, cp_rank, sp,
                        qkv_mode=1 if layout == "grouped" else 2, q_per_group=g, hq=hq, hk=hk, freqs_k=fk)
        return out
    # composed path: the plain rotation on the query and key views
    out = x_sbhd if inplace else x_sbhd.clone()
    s_, b_, _, d = x_sbhd.shape
    if layout == "grouped":
        v5 = out.unflatten(2, (hk, g + 2))   # always a view: the rotated heads are written back through it
        qv, kv = v5[:, :, :, :g].reshape(s_, b_, hq, d), v5[:, :, :, g]
        q_new = rope_apply(qv, q_freqs, interleaved=interleaved, backward=backward, cp_size=cp_size, cp_rank=cp_rank,
                           start_positions=start_positions)
        k_new = rope_apply(kv, k_freqs, interleaved=interleaved, backward=backward, cp_size=cp_size, cp_rank=cp_rank,
                           start_positions=start_positions)
        v5[:, :, :, :g].copy_(q_new.reshape(s_, b_, hk, g, d))
        v5[:, :, :, g].copy_(k_new)
    else:
        q_new = rope_apply(out[:, :, :hq], q_freqs, interleaved=interleaved, backward=backward, cp_size=cp_size,
                           cp_rank=cp_rank, start_positions=start_positions)
        k_new = rope_apply(out[:, :, hq:hq + hk], k_freqs, interleaved=interleaved, backward=backward, cp_size=cp_size,
                           cp_rank=cp_rank, start_positions=start_positions)
        out[:, :, :hq].copy_(q_new)
        out[:, :, hq:hq + hk].copy_(k_new)
    return out


# ----------------------------------------------------------------------------- cross entropy
def cross_entropy_ref(logits, targets, label_smoothing=0.0, ignore_index=-100):
    lf = logits.float().reshape(-1, logits.shape[-1])
    t = targets.reshape(-1)
    lse = torch.logsumexp(lf, dim=-1)
    safe_t = t.clamp(min=0)
    nll = lse - lf.gather(1, safe_t[:, None]).squeeze(1)
    if label_smoothing > 0:
        smooth = lse - lf.mean(-1)
        nll = (1 - label_smoothing) * nll + label_smoothing * smooth
    return torch.where(t == ignore_index, torch.zeros_like(nll), nll)


def cross_entropy_fwd_bwd(logits: torch.Tensor, targets: torch.Tensor, grad_scale: float = 1.0,
                          label_smoothing: float = 0.0, ignore_index: int = -100, inplace_grad: bool = True):
    """Per-row loss (fp32 ``[R]``) and d(loss)/d(logits)*grad_scale (written over the logits when
    ``inplace_grad``)."""
    V = logits.shape[-1]
    l2 = logits.reshape(-1, V)
    t = targets.reshape(-1).to(torch.int64)
    if _ext.use_cuda(logits) and label_smoothing == 0.0 and l2.stride(-1) == 1 \
            and logits.dtype in (torch.bfloat16, torch.float16, torch.float32):
        loss = torch.empty(l2.shape[0], dtype=torch.float32, device=logits.device)
        grad = l2 if inplace_grad else torch.empty_like(l2)
        _ext.get().cross_entropy(l2, t.contiguous(), loss, grad, None, None, None, 0, grad_scale, label_smoothing,
                                 ignore_index, None, None, None)
        return loss, grad.reshape(logits.shape)
    lf = l2.float()
    loss = cross_entropy_ref(lf, t, label_smoothing, ignore_index)
    p = torch.softmax(lf, dim=-1)
    p = p - label_smoothing / V
    p[torch.arange(p.shape[0], device=p.device), t.clamp(min=0)] -= 1 - label_smoothing
    p = torch.where((t == ignore_index)[:, None], torch.zeros_like(p), p) * grad_scale
    return loss, p.to(logits.dtype).reshape(logits.shape)


def cross_entropy_stats(logits, targets, vocab_start, ignore_index=-100):
    """Vocab-parallel stage 1: per-row (max, sum-exp, target logit or 0) of the local shard."""
    V = logits.shape[-1]
    l2 = logits.reshape(-1, V)
    t = targets.reshape(-1).to(torch.int64)
    R = l2.shape[0]
    if _ext.use_cuda(logits) and l2.stride(-1) == 1:
        st = torch.empty(3, R, dtype=torch.float32, device=logits.device)
        _ext.get().cross_entropy(l2, t.contiguous(), None, None, st[0], st[1], st[2], vocab_start, 1.0, 0.0,
                                 ignore_index, None, None, None)
        return st[0], st[1], st[2]
    lf = l2.float()
    m = lf.max(-1).values
    s = torch.exp(lf - m[:, None]).sum(-1)
    local = t - vocab_start
    mine = (local >= 0) & (local < V) & (t != ignore_index)
    tl = torch.where(mine, lf.gather(1, local.clamp(0, V - 1)[:, None]).squeeze(1), torch.zeros_like(m))
    return m, s, tl


def cross_entropy_parallel_grad(logits, targets, gmax, gsum, vocab_start, grad_scale=1.0, ignore_index=-100,
                                inplace_grad=True, grad_scale_dev=None):
    """Vocab-parallel stage 2: gradient from the all-reduced statistics."""
    V = logits.shape[-1]
    l2 = logits.reshape(-1, V)
    t = targets.reshape(-1).to(torch.int64)
    if _ext.use_cuda(logits) and l2.stride(-1) == 1:
        grad = l2 if inplace_grad else torch.empty_like(l2)
        _ext.get().cross_entropy(l2, t.contiguous(), None, grad, None, None, None, vocab_start, grad_scale, 0.0,
                                 ignore_index, gmax.contiguous(), gsum.contiguous(),
                                 grad_scale_dev.float().reshape(1) if grad_scale_dev is not None else None)
        return grad.reshape(logits.shape)
    p = torch.exp(l2.float() - gmax[:, None]) / gsum[:, None]
    local = t - vocab_start
    mine = (local >= 0) & (local < V)
    rows = torch.arange(p.shape[0], device=p.device)[mine]
    p[rows, local[mine]] -= 1.0
    p = torch.where((t == ignore_index)[:, None], torch.zeros_like(p), p) * grad_scale
    if grad_scale_dev is not None:
        p = p * grad_scale_dev.float()
    return p.to(logits.dtype).reshape(logits.shape)


# ----------------------------------------------------------------------------- multi-tensor
def _filter_empty(lists):
    keep = [i for i, t in enumerate(lists[0]) if t.numel() > 0]
    return [[l[i] for i in keep] for l in lists]


def multi_tensor_adam(lists: Sequence[List[torch.Tensor]], lr, beta1, beta2, eps, step, adamw=True,
                      bias_correction=True, weight_decay=0.0, grad_scale=1.0, inv_scale=None, noop=None,
                      remainders: bool = False):
    """lists = [grads, params, exp_avg, exp_avg_sq (, master fp32 | int16 remainders)]; updates in place.

    ``step`` and ``lr`` may be device tensors (int32 / fp32 scalars): the kernel then reads them at run
    time, which keeps a launch captured in a CUDA graph valid for later steps.  With ``remainders`` the
    fifth list holds the low 16 bits of each fp32 weight and the bf16 parameter is its rounded high half
    (reference: ``store_param_remainders``, ``pytorch/optimizers/fused_adam.py:74-149``)."""
    lists = _filter_empty(lists)
    if not lists[0]:
        return
    step_t = step if isinstance(step, torch.Tensor) else None
    lr_t = lr if isinstance(lr, torch.Tensor) else None
    if _ext.use_cuda(lists[0][0]):
        _ext.get().multi_tensor_adam([list(l) for l in lists], 0.0 if lr_t is not None else float(lr), beta1, beta2,
                                     eps, 1 if step_t is not None else int(step), adamw, bias_correction,
                                     weight_decay, grad_scale, inv_scale, noop, MT_CHUNK, step_t, lr_t, remainders)
        return
    if noop is not None and int(noop.item()) != 0:
        return
    step = int(step_t.item()) if step_t is not None else step
    lr = float(lr_t.item()) if lr_t is not None else lr
    bc1 = 1 - beta1 ** step if bias_correction else 1.0
    bc2 = 1 - beta2 ** step if bias_correction else 1.0
    gs = grad_scale * (float(inv_scale.item()) if inv_scale is not None else 1.0)
    has_master = len(lists) == 5 and not remainders
    for i in range(len(lists[0])):
        g = lists[0][i].float() * gs
        if remainders:
            p = join_param_remainder(lists[1][i], lists[4][i])
        else:
            p = lists[4][i] if has_master else lists[1][i].float()
        m, v = lists[2][i].float(), lists[3][i].float()
        if not adamw:
            g = g + weight_decay * p
        m = beta1 * m + (1 - beta1) * g
        v = beta2 * v + (1 - beta2) * g * g
        upd = (m / bc1) / (torch.sqrt(v / bc2) + eps)
        if adamw:
            upd = upd + weight_decay * p
        pn = p - lr * upd
        lists[2][i].copy_(m)
        lists[3][i].copy_(v)
        if remainders:
            hi, lo = split_param_remainder(pn)
            lists[1][i].copy_(hi)
            lists[4][i].copy_(lo)
            continue
        if has_master:
            lists[4][i].copy_(pn)
        lists[1][i].copy_(pn)


def split_param_remainder(w: torch.Tensor):
    """fp32 -> (bf16 parameter, int16 remainder): the remainder is the low half of the fp32 bits and the
    parameter the high half, incremented when the remainder is negative (round half up)."""
    u = w.contiguous().view(torch.int32)
    lo = (u & 0xFFFF).to(torch.int16)  # wraps to the signed low half
    hi = (u >> 16) + (lo < 0).to(torch.int32)
    return hi.to(torch.int16).view(torch.bfloat16), lo


def join_param_remainder(p_bf16: torch.Tensor, rem: torch.Tensor) -> torch.Tensor:
    hi = p_bf16.contiguous().view(torch.int16).to(torch.int32) - (rem < 0).to(torch.int32)
    return ((hi << 16) | (rem.to(torch.int32) & 0xFFFF)).view(torch.float32)


def multi_tensor_sgd(lists, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, first_run=False,
                     wd_after_momentum=False, grad_scale=1.0, noop=None):
    """lists = [grads, params, momentum_buf fp32 (, master fp32)]."""
    lists = _filter_empty(lists)
    if not lists[0]:
        return
    if _ext.use_cuda(lists[0][0]):
        _ext.get().multi_tensor_sgd([list(l) for l in lists], lr, momentum, dampening, weight_decay, nesterov,
                                    first_run, wd_after_momentum, grad_scale, noop, MT_CHUNK)
        return
    has_master = len(lists) == 4
    for i in range(len(lists[0])):
        g = lists[0][i].float() * grad_scale
        w = lists[3][i] if has_master else lists[1][i].float()
        if weight_decay and not wd_after_momentum:
            g = g + weight_decay * w
        if momentum:
            b = g if first_run else lists[2][i] * momentum + (1 - dampening) * g
            lists[2][i].copy_(b)
            g = g + momentum * b if nesterov else b
        if weight_decay and wd_after_momentum:
            g = g + weight_decay * w
        wn = w - lr * g
        if has_master:
            lists[3][i].copy_(wn)
        lists[1][i].copy_(wn)


def multi_tensor_scale(lists, scale, noop=None):
    """lists = [src, dst]: dst = src * scale; sets ``noop`` to 1 on inf/nan input."""
    lists = _filter_empty(lists)
    if not lists[0]:
        return
    if _ext.use_cuda(lists[0][0]):
        _ext.get().multi_tensor_scale([list(l) for l in lists], scale, noop, MT_CHUNK)
        return
    for s, d in zip(*lists):
        if noop is not None and not torch.isfinite(s).all():
            noop.fill_(1)
        d.copy_(s.float() * scale)


def multi_tensor_l2norm(tensors: List[torch.Tensor], per_tensor: bool = False):
    """Returns (global L2 norm [1], per-tensor norms or None)."""
    tensors = [t for t in tensors if t.numel() > 0]
    if not tensors:
        z = torch.zeros(1)
        return z, (torch.zeros(0) if per_tensor else None)
    dev = tensors[0].device
    if _ext.use_cuda(tensors[0]):
        out = torch.zeros(1, dtype=torch.float32, device=dev)
        pt = torch.zeros(len(tensors), dtype=torch.float32, device=dev) if per_tensor else None
        by_dtype = {}
        for i, t in enumerate(tensors):
            by_dtype.setdefault(t.dtype, []).append((i, t))
        for dt, items in by_dtype.items():
            sub_pt = torch.zeros(len(items), dtype=torch.float32, device=dev) if per_tensor else None
            _ext.get().multi_tensor_l2norm_sq([[t.contiguous() for _, t in items]], out, sub_pt, MT_CHUNK)
            if per_tensor:
                pt[torch.tensor([i for i, _ in items], device=dev)] = sub_pt
        return out.sqrt(), (pt.sqrt() if per_tensor else None)
    sq = [t.float().pow(2).sum() for t in tensors]
    tot = torch.stack(sq).sum().sqrt().reshape(1)
    return tot, (torch.stack(sq).sqrt() if per_tensor else None)


# ----------------------------------------------------------------------------- softmax / dropout (unfused attention)
def scaled_masked_softmax(scores: torch.Tensor, mask: Optional[torch.Tensor], scale: float, causal: bool = False):
    """softmax(scale * scores + mask) over the last dim, fp32 accumulation; ``mask`` True = masked out.
    ``causal`` applies a bottom-right aligned upper-triangular mask."""
    if _ext.use_cuda(scores) and hasattr(_ext.get(), "softmax_fwd") and scores.dim() == 4 and \
            scores.dtype in (torch.float32, torch.bfloat16, torch.float16) and \
            (mask is None or (mask.dim() == 4 and mask.shape[1] == 1 and mask.shape[0] == scores.shape[0]
                              and mask.shape[2:] == scores.shape[2:])):
        m8 = None if mask is None else mask.to(torch.uint8).contiguous()
        return _ext.get().softmax_fwd(scores.contiguous(), m8, float(scale), bool(causal), scores.shape[2],
                                      scores.shape[1])
    s = scores.float() * scale
    if causal:
        sq, sk = s.shape[-2], s.shape[-1]
        tri = torch.ones(sq, sk, dtype=torch.bool, device=s.device).triu(diagonal=sk - sq + 1)
        s = s.masked_fill(tri, float("-inf"))
    if mask is not None:
        s = s.masked_fill(mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)  # fully masked rows
    return p.to(scores.dtype)


def softmax_bwd(probs: torch.Tensor, dprobs: torch.Tensor, scale: float) -> torch.Tensor:
    if _ext.use_cuda(probs) and hasattr(_ext.get(), "softmax_bwd") and probs.dtype == dprobs.dtype and \
            probs.dtype in (torch.float32, torch.bfloat16, torch.float16):
        return _ext.get().softmax_bwd(probs.contiguous(), dprobs.contiguous(), float(scale))
    p, d = probs.float(), dprobs.float()
    return ((d - (d * p).sum(-1, keepdim=True)) * p * scale).to(probs.dtype)


def dropout_fwd(x: torch.Tensor, p: float, generator=None):
    """Returns (y, keep mask as bool)."""
    if p <= 0.0:
        return x, None
    if _ext.use_cuda(x) and hasattr(_ext.get(), "dropout_fwd") and generator is None and \
            x.dtype in (torch.float32, torch.bfloat16, torch.float16):
        seed = int(torch.cuda.initial_seed()) & 0x7FFFFFFFFFFFFFFF
        offset = int(torch.randint(0, 2**31 - 1, (1,)).item())  # advances the host generator: a new mask per call
        y, bits = _ext.get().dropout_fwd(x.contiguous(), float(p), seed, offset)
        return y, bits
    keep = torch.rand(x.shape, device=x.device, generator=generator) >= p
    return (x.float() * keep / (1 - p)).to(x.dtype), keep


def dropout_bwd(dy: torch.Tensor, keep: Optional[torch.Tensor], p: float):
    if keep is None:
        return dy
    if keep.dtype == torch.uint8 and _ext.use_cuda(dy):  # packed keep-bits from the CUDA forward
        return _ext.get().dropout_bwd(dy.contiguous(), keep, float(p))
    return (dy.float() * keep / (1 - p)).to(dy.dtype)


# ----------------------------------------------------------------------------- column sums, offsets, padding
def column_sum(x2d: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """``out[c] = sum_r x[r, c]`` in fp32 (the bias gradient of a linear layer); deterministic."""
    out_dtype = out_dtype or x2d.dtype
    if _ext.use_cuda(x2d) and x2d.dim() == 2 and x2d.stride(1) == 1 and x2d.shape[1] % 8 == 0 \
            and x2d.dtype in (torch.bfloat16, torch.float16, torch.float32) \
            and out_dtype in (torch.bfloat16, torch.float16, torch.float32) \
            and x2d.data_ptr() % 16 == 0 and (x2d.stride(0) * x2d.element_size()) % 16 == 0:
        return _ext.get().column_sum(x2d, out_dtype)
    return x2d.float().sum(dim=0).to(out_dtype)


def _vec_ok(t: torch.Tensor) -> bool:
    return (_ext.use_cuda(t) and t.dim() == 2 and t.stride(1) == 1 and t.shape[1] % 8 == 0
            and t.dtype in (torch.bfloat16, torch.float16, torch.float32) and t.data_ptr() % 16 == 0
            and (t.stride(0) * t.element_size()) % 16 == 0)


def grouped_column_sum(x2d: torch.Tensor, offsets: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """Per-slab column sums ``out[g] = x[offsets[g]:offsets[g+1]].sum(0)`` (the bias gradients of a grouped linear
    layer) in one launch; ``offsets``: int32 tensor of ``groups + 1`` row offsets."""
    out_dtype = out_dtype or x2d.dtype
    if _vec_ok(x2d) and offsets.is_cuda and (out_dtype == x2d.dtype or out_dtype == torch.float32):
        return _ext.get().grouped_column_sum(x2d, offsets.to(torch.int32).contiguous(), out_dtype)
    o = [int(v) for v in offsets.tolist()]
    return torch.stack([x2d[o[g]:o[g + 1]].float().sum(0) for g in range(len(o) - 1)]).to(out_dtype)


def grouped_bias_add_(x2d: torch.Tensor, bias_gc: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """``x[offsets[g]:offsets[g+1]] += bias[g]`` for every slab, in place, one launch."""
    if _ext.use_cuda(x2d) and x2d.dim() == 2 and x2d.stride(1) == 1 and offsets.is_cuda \
            and x2d.dtype in (torch.bfloat16, torch.float16, torch.float32):
        _ext.get().grouped_bias_add(x2d, bias_gc.to(x2d.dtype).contiguous(), offsets.to(torch.int32).contiguous())
        return x2d
    o = [int(v) for v in offsets.tolist()]
    for g in range(len(o) - 1):
        if o[g + 1] > o[g]:
            x2d[o[g]:o[g + 1]] += bias_gc[g].to(x2d.dtype)
    return x2d


def row_dot(a2d: torch.Tensor, b2d: torch.Tensor) -> torch.Tensor:
    """``out[r] = <a[r], b[r]>`` in fp32: one pass over both operands (gradient of a per-row scale)."""
    if _vec_ok(a2d) and _vec_ok(b2d) and a2d.dtype == b2d.dtype and a2d.shape == b2d.shape:
        return _ext.get().row_dot(a2d, b2d)
    return (a2d.float() * b2d.float()).sum(-1)


def splits_to_offsets(splits: torch.Tensor, multiplier: int = 1, dtype=torch.int32) -> torch.Tensor:
    """Exclusive prefix sums ``[0, s0, s0 + s1, ...] * multiplier`` of a device tensor of split sizes, without a
    host round trip (reference: ``common/util/splits_to_offsets.cu:61``)."""
    assert dtype in (torch.int32, torch.int64)
    if _ext.use_cuda(splits) and splits.dtype in (torch.int32, torch.int64) and splits.dim() == 1:
        return _ext.get().splits_to_offsets(splits.contiguous(), int(multiplier), dtype == torch.int64)
    z = torch.zeros(1, dtype=torch.int64, device=splits.device)
    return (torch.cat([z, torch.cumsum(splits.to(torch.int64), 0)]) * int(multiplier)).to(dtype)


def repad_rows(x2d: torch.Tensor, in_splits, out_splits) -> torch.Tensor:
    """Copy row slabs of sizes ``in_splits`` into slabs of sizes ``out_splits``: longer slabs are zero-filled at
    their end (padding for FP8 alignment), shorter ones cut (unpadding).  Splits are lists of ints or device
    tensors; one launch for all slabs (reference: ``common/util/padding.cu:46,130``)."""
    host = not isinstance(in_splits, torch.Tensor)
    if host:
        ins = torch.tensor(list(in_splits), dtype=torch.int32)
        outs = torch.tensor(list(out_splits), dtype=torch.int32)
        out_rows = int(outs.sum())
    else:
        ins, outs = in_splits, out_splits
        out_rows = None
    if _ext.use_cuda(x2d) and x2d.dim() == 2 and (x2d.shape[1] * x2d.element_size()) % 16 == 0:
        z = torch.zeros(1, dtype=torch.int32)
        if host:
            io = torch.cat([z, torch.cumsum(ins, 0).to(torch.int32)]).to(x2d.device, non_blocking=True)
            oo = torch.cat([z, torch.cumsum(outs, 0).to(torch.int32)]).to(x2d.device, non_blocking=True)
        else:
            io, oo = splits_to_offsets(ins.to(x2d.device)), splits_to_offsets(outs.to(x2d.device))
            out_rows = int(outs.sum())  # the result's shape is host data: device splits cost one read here
        return _ext.get().repad_rows(x2d.contiguous(), io, oo, out_rows)
    il = [int(v) for v in (ins.tolist())]
    ol = [int(v) for v in (outs.tolist())]
    chunks = torch.split(x2d, il, dim=0)
    res = []
    for c, m, p in zip(chunks, il, ol):
        res.append(c[:p] if p <= m else torch.nn.functional.pad(c, (0, 0, 0, p - m)))
    return torch.cat(res, dim=0) if res else x2d[:0]


def pad_last_dim(x: torch.Tensor, new_cols: int) -> torch.Tensor:
    """Zero-pad (or cut) the last dimension to ``new_cols`` (head-dim padding of block-scaled attention inputs)."""
    C = x.shape[-1]
    if new_cols == C:
        return x
    if _ext.use_cuda(x) and (C * x.element_size()) % 4 == 0 and (new_cols * x.element_size()) % 4 == 0:
        return _ext.get().pad_last_dim(x.contiguous(), int(new_cols))
    return x[..., :new_cols] if new_cols < C else torch.nn.functional.pad(x, (0, new_cols - C))
