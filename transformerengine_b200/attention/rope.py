"""Rotary position embeddings (reference: ``pytorch/attention/rope.py:18-345``)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class RotaryPositionEmbedding(torch.nn.Module):
    """Produces the angle table ``[seq, 1, 1, dim]`` (fp32) consumed by :func:`apply_rotary_pos_emb`."""

    def __init__(self, dim: int, rotary_percent: float = 1.0, seq_len_interpolation_factor: Optional[int] = None,
                 pretrained_max_position_embeddings: Optional[int] = None, rotary_base: float = 10000.0,
                 interleaved: bool = False):
        super().__init__()
        if rotary_percent < 1.0:
            dim = int(dim * rotary_percent)
        self.dim = dim
        self.seq_len_interpolation_factor = seq_len_interpolation_factor
        self.rotary_base = rotary_base
        self.pretrained_max_position_embeddings = pretrained_max_position_embeddings
        self.interleaved = interleaved

    def forward(self, max_seq_len: int, offset: int = 0) -> torch.Tensor:
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        seq = torch.arange(max_seq_len, device=dev, dtype=torch.float32) + offset
        if self.pretrained_max_position_embeddings is not None and self.seq_len_interpolation_factor is not None:
            if max_seq_len > self.pretrained_max_position_embeddings * self.seq_len_interpolation_factor:
                seq = seq * (self.pretrained_max_position_embeddings / max_seq_len)
            else:
                seq = seq / self.seq_len_interpolation_factor
        emb = ops.rope_freqs(seq, self.dim, self.rotary_base, self.interleaved)
        return emb.reshape(emb.shape[0], 1, 1, emb.shape[1])


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, freqs, fmt, interleaved, cp_size, cp_rank, start_positions):  # type: ignore[override]
        x = t if fmt == "sbhd" else t.transpose(0, 1)
        f = freqs.reshape(freqs.shape[0], freqs.shape[-1])
        y = ops.rope_apply(x, f, interleaved=interleaved, cp_size=cp_size, cp_rank=cp_rank,
                           start_positions=start_positions)
        ctx.save_for_backward(f, start_positions if start_positions is not None else torch.empty(0))
        ctx.cfg = (fmt, interleaved, cp_size, cp_rank, start_positions is not None)
        return y if fmt == "sbhd" else y.transpose(0, 1)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        f, sp = ctx.saved_tensors
        fmt, interleaved, cp_size, cp_rank, has_sp = ctx.cfg
        x = g if fmt == "sbhd" else g.transpose(0, 1)
        if x.stride(-1) != 1:
            x = x.contiguous()
        y = ops.rope_apply(x, f, interleaved=interleaved, backward=True, cp_size=cp_size, cp_rank=cp_rank,
                           start_positions=sp if has_sp else None)
        return (y if fmt == "sbhd" else y.transpose(0, 1)), None, None, None, None, None, None


def apply_rotary_pos_emb(t: torch.Tensor, freqs: torch.Tensor, tensor_format: str = "sbhd",
                         start_positions: Optional[torch.Tensor] = None, interleaved: bool = False,
                         fused: bool = True, cu_seqlens: Optional[torch.Tensor] = None, cp_size: int = 1,
                         cp_rank: int = 0) -> torch.Tensor:
    """Rotate the first ``freqs.shape[-1]`` channels of ``t`` (``sbhd``, ``bshd`` or ``thd``).  ``fused=False``
    selects the plain PyTorch formula (differentiated by autograd) instead of the kernel."""
    if not fused and tensor_format in ("sbhd", "bshd") and cp_size == 1:
        x = t if tensor_format == "sbhd" else t.transpose(0, 1)
        f = freqs.reshape(freqs.shape[0], freqs.shape[-1])
        y = ops.misc.rope_ref(x, f.float(), f.shape[-1], interleaved, False, 0, 1, 0, start_positions)
        return y if tensor_format == "sbhd" else y.transpose(0, 1)
    if tensor_format == "thd":
        assert cu_seqlens is not None, "thd format needs cu_seqlens"
        outs = []
        cs = cu_seqlens.tolist()
        for i in range(len(cs) - 1):
            seg = t[cs[i] // cp_size:cs[i + 1] // cp_size].unsqueeze(1)  # [s,1,h,d]
            outs.append(_RopeFn.apply(seg, freqs, "sbhd", interleaved, cp_size, cp_rank, None).squeeze(1))
        return torch.cat(outs, dim=0)
    assert tensor_format in ("sbhd", "bshd")
    return _RopeFn.apply(t, freqs, tensor_format, interleaved, cp_size, cp_rank, start_positions)


class _RopeQkvFn(torch.autograd.Function):
    """Rotation of the query and key heads of a packed QKV projection, in place, one launch."""

    @staticmethod
    def forward(ctx, mixed, q_freqs, k_freqs, fmt, layout, hq, hk, d, interleaved, cp_size, cp_rank, start_positions,
                inplace):  # type: ignore[override]
        lead = mixed.shape[:2]
        x4 = mixed.view(*lead, hq + 2 * hk, d)
        x = x4 if fmt == "sbhd" else x4.transpose(0, 1)
        fq = q_freqs.reshape(q_freqs.shape[0], q_freqs.shape[-1])
        fk = fq if k_freqs is q_freqs else k_freqs.reshape(k_freqs.shape[0], k_freqs.shape[-1])
        y = ops.rope_qkv(x, fq, fk, layout=layout, hq=hq, hk=hk, interleaved=interleaved, cp_size=cp_size,
                         cp_rank=cp_rank, start_positions=start_positions, inplace=inplace)
        ctx.save_for_backward(fq, fk, start_positions if start_positions is not None else torch.empty(0))
        ctx.cfg = (fmt, layout, hq, hk, d, interleaved, cp_size, cp_rank, start_positions is not None)
        if inplace:
            ctx.mark_dirty(mixed)
            return mixed
        y = y if fmt == "sbhd" else y.transpose(0, 1)
        return y.reshape(mixed.shape)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        fq, fk, sp = ctx.saved_tensors
        fmt, layout, hq, hk, d, interleaved, cp_size, cp_rank, has_sp = ctx.cfg
        g = g.contiguous()
        g4 = g.view(*g.shape[:2], hq + 2 * hk, d)
        x = g4 if fmt == "sbhd" else g4.transpose(0, 1)
        # out of place: the incoming gradient may be shared with other consumers
        y = ops.rope_qkv(x, fq, fq if fk is fq else fk, layout=layout, hq=hq, hk=hk, interleaved=interleaved, backward=True,
                         cp_size=cp_size, cp_rank=cp_rank, start_positions=sp if has_sp else None)
        y = y if fmt == "sbhd" else y.transpose(0, 1)
        return (y.reshape(g.shape),) + (None,) * 12


def rotate_packed_qkv_(mixed: torch.Tensor, q_freqs: torch.Tensor, k_freqs: torch.Tensor, tensor_format: str, layout: str,
                       hq: int, hk: int, head_dim: int, *, interleaved: bool = False, cp_size: int = 1, cp_rank: int = 0,
                       start_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate the query and key heads of ``mixed`` (``[s, b, (hq + 2 hk) * d]`` or ``[b, s, ...]``, the output of a
    fused QKV projection) with one kernel launch and return the result; value heads pass through.  The rotation
    runs in place when autograd allows it (``mixed`` is not a view made inside another function), else into a new
    tensor.  ``layout``: ``"grouped"`` (per key/value group: its query heads, the key head, the value head) or
    ``"blocked"`` (all queries, all keys, all values)."""
    assert mixed.dim() == 3 and mixed.is_contiguous() and mixed.shape[-1] == (hq + 2 * hk) * head_dim
    inplace = not mixed._is_view() and not (mixed.is_leaf and mixed.requires_grad)
    return _RopeQkvFn.apply(mixed, q_freqs, k_freqs, tensor_format, layout, hq, hk, head_dim, interleaved, cp_size,
                            cp_rank, start_positions, inplace)


def apply_fused_qkv_rotary_pos_emb(qkv: torch.Tensor, q_freqs: torch.Tensor, k_freqs: torch.Tensor,
                                   qkv_split_arg_list, tensor_format: str = "sbhd",
                                   start_positions: Optional[torch.Tensor] = None, interleaved: bool = False,
                                   cu_seqlens: Optional[torch.Tensor] = None, cp_size: int = 1, cp_rank: int = 0):
    """Split a packed QKV projection and rotate Q and K.

    ``qkv`` is ``[s, b, g, q + k + v]`` (or ``[b, s, ...]``) with, per key/value group ``g``, ``q`` query
    channels (``q / d`` heads), ``k`` key channels and ``v = d`` value channels
    (``qkv_split_arg_list = [q, k, v]``).  Returns ``(q [.., g * q/d, d], k [.., g * k/d, d], v [.., g, d])``
    with the rotation applied to Q and K.  With one key head per group (the usual GQA packing) split and both
    rotations are one kernel launch; other packings rotate Q and K separately.
    (Reference: ``pytorch/attention/rope.py:465``.)"""
    assert tensor_format in ("sbhd", "bshd") and len(qkv_split_arg_list) == 3
    nq, nk, nv = (int(x) for x in qkv_split_arg_list)
    assert qkv.shape[-1] == nq + nk + nv and nq % nv == 0 and nk % nv == 0, "split sizes must be whole heads"
    d = nv
    if nk == nv and qkv.dim() == 4 and qkv.is_contiguous() and cu_seqlens is None:
        # one key and one value head per group: the packed tensor is the "grouped" head layout of the kernel
        g, qpg = qkv.shape[2], nq // d
        flat = qkv.reshape(qkv.shape[0], qkv.shape[1], -1)
        rot = _RopeQkvFn.apply(flat, q_freqs, k_freqs, tensor_format, "grouped", g * qpg, g, d, interleaved, cp_size,
                               cp_rank, start_positions, False)
        rot = rot.reshape(*qkv.shape[:2], g, qpg + 2, d)
        q, k, v = torch.split(rot, (qpg, 1, 1), dim=-2)
        return (q.reshape(*qkv.shape[:2], g * qpg, d), k.reshape(*qkv.shape[:2], g, d), v.reshape(*qkv.shape[:2], g, d))
    q, k, v = torch.split(qkv, [nq, nk, nv], dim=-1)
    lead = qkv.shape[:2]
    q = q.reshape(*lead, -1, d)
    k = k.reshape(*lead, -1, d)
    q = apply_rotary_pos_emb(q, q_freqs, tensor_format, start_positions=start_positions, interleaved=interleaved,
                             cp_size=cp_size, cp_rank=cp_rank)
    k = apply_rotary_pos_emb(k, k_freqs, tensor_format, start_positions=start_positions, interleaved=interleaved,
                             cp_size=cp_size, cp_rank=cp_rank)
    return q, k, v


# names of the reference's autograd functions (``pytorch/attention/rope.py``) for code that calls ``.apply`` on them
FusedRoPEFunc = _RopeFn
FusedQKVRoPEFunc = _RopeQkvFn
