"""Context-parallel ring attention over packed ("thd") sequences.

Every sequence is cut into ``2 * cp`` chunks and rank ``r`` holds chunks ``r`` and ``2 * cp - 1 - r``
of EVERY sequence (``attention.thd.thd_get_partitioned_indices``), so causal work is balanced.  K/V
shards travel around the ring; with a causal mask a step is one of three products:

* own K/V: all local queries, causal mask;
* K/V of an earlier rank: all local queries against the FIRST half of that rank's K/V, no mask
  (its second chunk lies after every local query);
* K/V of a later rank: the SECOND half of the local queries against all of that K/V, no mask
  (the first local chunk precedes both of its chunks).

Partial outputs are merged through their log-sum-exp with the packed-sequence kernels
(``thd_out_correction``, ``thd_second_half_lse_correction``); the backward replays the steps with the
merged statistics and sends dK/dV around the ring with their shard.  Each product is one launch of the
variable-length attention kernels on the GPU, or the fp32 reference math per sequence elsewhere.
(Reference: ``pytorch/attention/dot_product_attention/context_parallel.py``, thd branches of
``AttnFuncWithCPAndKVP2P``.)
"""
from __future__ import annotations

import importlib
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..attention import thd
from ..ops import _ext, flash
from .context_parallel import _block_bwd, _block_fwd, _ring_exchange


_attention_module = importlib.import_module(flash.__name__.rsplit(".", 1)[0] + ".attention")


def _use_kernels(q, k, v) -> bool:
    return q.is_cuda and _attention_module._USE_OWN_FLASH and flash.supported_varlen(q, k, v)


class _SeqMap:
    """Token -> (sequence, position) maps of a packed layout, for moving LSE between the packed
    ``[h, t]`` form of the merge kernels and the ``[sequences, h, s_pad]`` form of the attention kernels."""

    def __init__(self, cu: torch.Tensor, t: int, max_len: int):
        self.cu, self.t, self.max_len = cu, t, max_len
        self.nseq = cu.numel() - 1
        tok = torch.arange(t, device=cu.device)
        seq = torch.searchsorted(cu[1:].contiguous(), tok, right=True).clamp_(max=self.nseq - 1)
        pos = tok - cu[seq.long()].long()
        valid = (tok < cu[-1]) & (pos < max_len)
        # tokens after the last sequence go to a scratch row past the real sequences
        self.seq = torch.where(valid, seq, torch.full_like(seq, self.nseq))
        self.pos = torch.where(valid, pos, torch.zeros_like(pos))
        self.s_pad = (max_len + 127) // 128 * 128

    def to_padded(self, lse_packed: torch.Tensor) -> torch.Tensor:
        out = lse_packed.new_zeros(self.nseq + 1, lse_packed.shape[0], self.s_pad)
        out[self.seq, :, self.pos] = lse_packed.t()
        return out[:self.nseq]

    def to_packed(self, lse_padded: torch.Tensor) -> torch.Tensor:
        scratch = lse_padded.new_full((1,) + tuple(lse_padded.shape[1:]), float("-inf"))
        return torch.cat([lse_padded, scratch])[self.seq, :, self.pos].t().contiguous()


def _half_cu(cu: torch.Tensor) -> torch.Tensor:
    return torch.div(cu, 2, rounding_mode="floor").to(cu.dtype)


def _block_fwd_thd(q, k, v, mq: _SeqMap, mk: _SeqMap, scale, causal) -> Tuple[torch.Tensor, torch.Tensor]:
    """One product over packed sequences: (out [tq, h, d] in q's dtype, lse [h, tq] fp32)."""
    if _use_kernels(q, k, v):
        C_ = _ext.get()
        out = torch.zeros_like(q)
        lse = torch.full((mq.nseq, q.shape[1], mq.s_pad), float("-inf"), dtype=torch.float32, device=q.device)
        C_.flash_fwd_varlen(flash._thd_view(q), flash._thd_view(k), flash._thd_view(v), flash._thd_view(out), lse,
                            mq.cu, mk.cu, mq.cu, mk.cu, mq.max_len, mk.max_len, float(scale), bool(causal), True,
                            C_.status(q.device.index))
        return out, mq.to_packed(lse)
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    lse = torch.full((q.shape[1], q.shape[0]), float("-inf"), dtype=torch.float32, device=q.device)
    cq, ck = mq.cu.tolist(), mk.cu.tolist()
    for i in range(mq.nseq):
        a, b, c, e = cq[i], cq[i + 1], ck[i], ck[i + 1]
        if b == a or e == c:
            continue
        bh = lambda x: x.permute(1, 0, 2).unsqueeze(0)  # noqa: E731
        mask = None
        if causal:
            n, m = b - a, e - c
            mask = torch.arange(m, device=q.device)[None, :] > torch.arange(n, device=q.device)[:, None] + (m - n)
        o, l = _block_fwd(bh(q[a:b]), bh(k[c:e]), bh(v[c:e]), scale, mask)
        out[a:b] = o.squeeze(0).permute(1, 0, 2)
        lse[:, a:b] = l.squeeze(0)
    return out.to(q.dtype), lse


def _block_bwd_thd(do, q, k, v, o, lse_packed, mq: _SeqMap, mk: _SeqMap, scale, causal):
    """Gradients of one product given the MERGED output ``o`` and ``lse`` of the query tokens."""
    if _use_kernels(q, k, v):
        C_ = _ext.get()
        lse = mq.to_padded(lse_packed)
        delta = torch.empty_like(lse)
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        C_.flash_bwd_varlen(flash._thd_view(do.contiguous()), flash._thd_view(q), flash._thd_view(k),
                            flash._thd_view(v), flash._thd_view(o.contiguous()), lse, delta, flash._thd_view(dq),
                            flash._thd_view(dk), flash._thd_view(dv), mq.cu, mk.cu, mq.cu, mk.cu, mq.max_len,
                            mk.max_len, float(scale), bool(causal), True, C_.status(q.device.index))
        return dq, dk, dv
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    cq, ck = mq.cu.tolist(), mk.cu.tolist()
    for i in range(mq.nseq):
        a, b, c, e = cq[i], cq[i + 1], ck[i], ck[i + 1]
        if b == a or e == c:
            continue
        bh = lambda x: x.permute(1, 0, 2).unsqueeze(0)  # noqa: E731
        mask = None
        if causal:
            n, m = b - a, e - c
            mask = torch.arange(m, device=q.device)[None, :] > torch.arange(n, device=q.device)[:, None] + (m - n)
        g = _block_bwd(bh(do[a:b]), bh(q[a:b]), bh(k[c:e]), bh(v[c:e]), bh(o[a:b]), lse_packed[:, a:b].unsqueeze(0),
                       scale, mask)
        dq[a:b], dk[c:e], dv[c:e] = (x.squeeze(0).permute(1, 0, 2) for x in g)
    return dq, dk, dv


def _step_kind(causal: bool, me: int, src: int) -> str:
    if not causal:
        return "full"
    return "diag" if src == me else ("kv_first_half" if src < me else "q_second_half")


class _ThdRingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu, max_len, group, ranks, scale, causal):  # type: ignore[override]
        cp, me = dist.get_world_size(group), dist.get_rank(group)
        t = q.shape[0]
        full = _SeqMap(cu, t, max_len)
        half = _SeqMap(_half_cu(cu), t // 2, max_len // 2)
        kv = torch.stack([k, v]).contiguous()
        outs: List[Optional[torch.Tensor]] = []
        lses: List[Optional[torch.Tensor]] = []
        lse = None
        for step in range(cp):
            src = (me - step) % cp
            kind = _step_kind(causal, me, src)
            if kind in ("full", "diag"):
                o_s, l_s = _block_fwd_thd(q, kv[0], kv[1], full, full, scale, kind == "diag")
                lse = l_s.clone() if lse is None else torch.logaddexp(lse, l_s)
            elif kind == "kv_first_half":
                kvh = thd.thd_read_half_tensor(kv, cu, 0)
                o_s, l_s = _block_fwd_thd(q, kvh[0], kvh[1], full, half, scale, False)
                lse = torch.logaddexp(lse, l_s)
            else:
                qh = thd.thd_read_half_tensor(q, cu, 1)
                o_s, l_s = _block_fwd_thd(qh, kv[0], kv[1], half, full, scale, False)
                thd.thd_second_half_lse_correction(lse, l_s, cu)
            outs.append(o_s)
            lses.append(l_s)
            if step != cp - 1:
                kv = _ring_exchange(kv, group, ranks)
        out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        for step in range(cp):
            kind = _step_kind(causal, me, (me - step) % cp)
            thd.thd_out_correction(out, outs[step].float(), lse, lses[step], cu, kind == "q_second_half")
        o = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, o, lse, cu)
        ctx.cfg = (group, ranks, scale, causal, max_len)
        return o

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        q, k, v, o, lse, cu = ctx.saved_tensors
        group, ranks, scale, causal, max_len = ctx.cfg
        cp, me = dist.get_world_size(group), dist.get_rank(group)
        t = q.shape[0]
        full = _SeqMap(cu, t, max_len)
        half = _SeqMap(_half_cu(cu), t // 2, max_len // 2)
        do = do.contiguous()
        kv = torch.stack([k, v]).contiguous()
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        for step in range(cp):
            kind = _step_kind(causal, me, (me - step) % cp)
            if kind in ("full", "diag"):
                g = _block_bwd_thd(do, q, kv[0], kv[1], o, lse, full, full, scale, kind == "diag")
                dq += g[0].float()
                dkv[0] += g[1].float()
                dkv[1] += g[2].float()
            elif kind == "kv_first_half":
                kvh = thd.thd_read_half_tensor(kv, cu, 0)
                g = _block_bwd_thd(do, q, kvh[0], kvh[1], o, lse, full, half, scale, False)
                dq += g[0].float()
                thd.thd_grad_correction(dkv, torch.stack([g[1], g[2]]).float(), cu, "add", "none")
            else:
                qh, doh, oh = (thd.thd_read_half_tensor(x, cu, 1) for x in (q, do, o))
                lse_h = thd.thd_read_second_half_lse(lse, cu)
                g = _block_bwd_thd(doh, qh, kv[0], kv[1], oh, lse_h, half, full, scale, False)
                thd.thd_grad_correction(dq, g[0].float().contiguous(), cu, "none", "add")
                dkv[0] += g[1].float()
                dkv[1] += g[2].float()
            # gradients travel with their K/V shard; after cp hops they are back at the owner
            if cp > 1:
                dkv = _ring_exchange(dkv, group, ranks)
                if step != cp - 1:
                    kv = _ring_exchange(kv, group, ranks)
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None, None, None


def thd_ring_attention(q, k, v, cu_seqlens, *, cp_group, scale: Optional[float] = None, causal: bool = True,
                       cp_global_ranks=None, max_seqlen: Optional[int] = None) -> torch.Tensor:
    """Attention over packed sequences sharded over ``cp_group``.

    ``q`` / ``k`` / ``v`` are this rank's tokens ``[t_local, h, d]`` in the dual-chunk layout,
    ``cu_seqlens`` the cumulative LOCAL lengths (global lengths divided by the group size; every local
    length must be even).  Returns ``[t_local, h, d]``."""
    cu = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
    assert q.shape[0] % 2 == 0 and k.shape[0] == q.shape[0], "self-attention over an even number of local tokens"
    if max_seqlen is None:
        max_seqlen = int((cu[1:] - cu[:-1]).max())
    max_seqlen += max_seqlen % 2
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    return _ThdRingAttention.apply(q, k, v, cu, int(max_seqlen), cp_group, cp_global_ranks, float(scale), causal)
