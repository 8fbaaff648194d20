"""Context parallelism: attention over a sequence that is sharded across ranks.

Communication types (reference: ``pytorch/attention/dot_product_attention/
context_parallel.py:1356, 3014, 4170, 4924``):

* ``"p2p"``        ring exchange of K/V blocks with online-softmax (LSE) merging;
* ``"all_gather"`` gather all K/V, attend locally;
* ``"a2a"``        Ulysses: all-to-all trades the sequence shard for a head shard.

For causal masks the sequence is expected in the load-balanced "dual chunk" order: the
sequence is cut in ``2*cp`` chunks and rank ``r`` holds chunks ``r`` and ``2*cp-1-r``
(:func:`get_batch_on_this_cp_rank`).  Masks are derived from global token positions, so any
chunk order works.  Tensors are ``[b, h, s_local, d]``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------- layout helpers
def dual_chunk_positions(s_local: int, cp_size: int, cp_rank: int, device=None) -> torch.Tensor:
    """Global positions of this rank's tokens in the dual-chunk layout."""
    half = s_local // 2
    a = torch.arange(half, device=device)
    return torch.cat([a + cp_rank * half, a + (2 * cp_size - 1 - cp_rank) * half])


def get_batch_on_this_cp_rank(x: torch.Tensor, cp_size=None, cp_rank=None, seq_dim=1, cp_group=None,
                              qvk_format: str = "thd"):
    """Slice a full-sequence tensor to the two chunks owned by ``cp_rank``: ``(x, cp_size, cp_rank, seq_dim)``.

    Reference call form for packed batches, ``(cu_seqlens_padded, input_ids_padded, labels_padded,
    position_ids_padded, cp_group=None, qvk_format="thd")``: every sequence (padded to a multiple of ``2 * cp``)
    gives this rank its chunk ``r`` and its chunk ``2 * cp - 1 - r``; returns the three sliced tensors."""
    if isinstance(cp_size, torch.Tensor) or (cp_size is None and cp_rank is None):
        return _thd_batch_on_this_cp_rank(x, cp_size, cp_rank, seq_dim if isinstance(seq_dim, torch.Tensor) else None,
                                          cp_group, qvk_format)
    if cp_size == 1:
        return x
    chunks = x.chunk(2 * cp_size, dim=seq_dim)
    return torch.cat([chunks[cp_rank], chunks[2 * cp_size - 1 - cp_rank]], dim=seq_dim)


def _natural_order_index(half: int, cp_size: int, device=None) -> torch.Tensor:
    """Index that reorders a sequence stored as the ranks' dual-chunk shards back to back (rank 0's two
    chunks, rank 1's two chunks, ...) into natural token order: ``natural = stored.index_select(dim, idx)``."""
    slot = [0] * (2 * cp_size)  # slot[c] = where chunk c sits in the stored order
    for r in range(cp_size):
        slot[r] = 2 * r
        slot[2 * cp_size - 1 - r] = 2 * r + 1
    a = torch.arange(half, device=device)
    return torch.cat([a + slot[c] * half for c in range(2 * cp_size)])


def _thd_batch_on_this_cp_rank(cu_seqlens_padded, input_ids, labels, position_ids, cp_group, qvk_format):
    if qvk_format not in ("thd", "bshd", "sbhd"):
        raise ValueError(f"Unsupported qvk_format: {qvk_format}!")
    if qvk_format != "thd":
        raise ValueError(f"Support not implemented yet for qvk_format: {qvk_format}!")
    cp = dist.get_world_size(cp_group) if dist.is_initialized() else 1
    if cp == 1:
        return input_ids, labels, position_ids
    rank = dist.get_rank(cp_group)
    total = int(cu_seqlens_padded[-1])
    starts = cu_seqlens_padded[:-1].tolist()
    sizes = ((cu_seqlens_padded[1:] - cu_seqlens_padded[:-1]) // (2 * cp)).tolist()
    pieces = []
    for st, n in zip(starts, sizes):
        pieces.append(torch.arange(st + rank * n, st + (rank + 1) * n))
        pieces.append(torch.arange(st + (2 * cp - 1 - rank) * n, st + (2 * cp - rank) * n))
    idx = torch.cat(pieces)

    def cut(t):
        if t is None:
            return None
        if t.dim() == 1:
            dim = 0
        elif t.shape[1] == total:
            dim = 1
        elif t.shape[0] == total:
            dim = 0
        else:
            raise ValueError("Make sure the inputs are in THD format and padded correctly.")
        if t.shape[dim] != total:
            raise ValueError("the tensor's token dimension does not match cu_seqlens_padded[-1]")
        return t.index_select(dim, idx.to(t.device))

    return cut(input_ids), cut(labels), cut(position_ids)


def generate_positional_ids_for_cp(cu_seqlens: torch.Tensor, divisibility_factor: int,
                                   dtype: torch.dtype = torch.long) -> torch.Tensor:
    """Position ids of a packed batch whose sequences are padded to multiples of ``divisibility_factor``: every
    sequence counts from 0 through its padding."""
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    f = divisibility_factor
    return torch.cat([torch.arange(-(-n // f) * f, dtype=dtype) for n in lens])


def pad_thd_sequences_for_cp(cu_seqlens: torch.Tensor, cp_size=None, *rest, **kw):
    """Cumulative lengths after padding every sequence to a multiple of ``2*cp``: ``(cu_seqlens, cp_size)``.

    Reference call form ``(input_ids, labels, cu_seqlens, divisibility_factor, padding_token_id=0,
    padding_label_id=-100)``: pads the packed tokens and labels themselves and returns
    ``(input_ids_padded, labels_padded, cu_seqlens_padded)``."""
    if isinstance(cp_size, torch.Tensor):
        return _pad_thd_tokens(cu_seqlens, cp_size, *rest, **kw)
    lens = cu_seqlens[1:] - cu_seqlens[:-1]
    m = 2 * cp_size
    padded = (lens + m - 1) // m * m
    out = torch.zeros_like(cu_seqlens)
    out[1:] = padded.cumsum(0)
    return out


def _pad_thd_tokens(input_ids, labels, cu_seqlens, divisibility_factor, padding_token_id: int = 0,
                    padding_label_id: int = -100):
    ids = input_ids.squeeze(0) if input_ids.dim() == 2 else input_ids
    lab = labels.squeeze(0) if labels.dim() == 2 else labels
    f = divisibility_factor
    bounds = cu_seqlens.tolist()
    out_ids, out_lab, new_cu = [], [], [0]
    for a, b in zip(bounds[:-1], bounds[1:]):
        pad = -(-(b - a) // f) * f - (b - a)
        out_ids += [ids[a:b], ids.new_full((pad,), padding_token_id)]
        out_lab += [lab[a:b], lab.new_full((pad,), padding_label_id)]
        new_cu.append(new_cu[-1] + b - a + pad)
    return torch.cat(out_ids), torch.cat(out_lab), torch.tensor(new_cu, dtype=cu_seqlens.dtype, device=cu_seqlens.device)


# --------------------------------------------------------------------------- block attention with explicit backward
def _block_fwd(q, k, v, scale, mask):
    """Returns (out fp32, lse) of one K/V block; ``mask`` True = masked out."""
    hq, hk = q.shape[1], k.shape[1]
    kf, vf = k.float(), v.float()
    if hk != hq:
        kf = kf.repeat_interleave(hq // hk, dim=1)
        vf = vf.repeat_interleave(hq // hk, dim=1)
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf), lse


def _block_bwd(do, q, k, v, o, lse, scale, mask):
    """Gradients of one block given the GLOBAL output ``o`` and log-sum-exp ``lse``."""
    hq, hk = q.shape[1], k.shape[1]
    rep = hq // hk
    kf, vf = k.float(), v.float()
    if rep > 1:
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(mask, float("-inf"))
    p = torch.nan_to_num(torch.exp(s - lse[..., None]), nan=0.0)
    dof = do.float()
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * o.float()).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), q.float())
    if rep > 1:
        b, _, sk, d = dk.shape
        dk = dk.reshape(b, hk, rep, sk, d).sum(2)
        dv = dv.reshape(b, hk, rep, sk, d).sum(2)
    return dq, dk, dv


def _mask_for(qpos, kpos, causal, window):
    if not causal and (window is None or (window[0] < 0 and window[1] < 0)):
        return None
    rel = kpos[None, :] - qpos[:, None]
    m = torch.zeros(rel.shape, dtype=torch.bool, device=qpos.device)
    right = 0 if causal else window[1]
    left = window[0] if window is not None else -1
    if right >= 0:
        m |= rel > right
    if left >= 0:
        m |= rel < -left
    return m


def _ring_exchange(t: torch.Tensor, group, ranks: Optional[List[int]]) -> torch.Tensor:
    """Send ``t`` to the next rank of the ring, receive from the previous one."""
    cp = dist.get_world_size(group)
    me = dist.get_rank(group)
    nxt, prv = (me + 1) % cp, (me - 1) % cp
    if ranks is not None:
        nxt, prv = ranks[nxt], ranks[prv]
    else:
        nxt, prv = dist.get_global_rank(group, nxt), dist.get_global_rank(group, prv)
    recv = torch.empty_like(t)
    ops = [dist.P2POp(dist.isend, t.contiguous(), nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]
    if me % 2:
        ops.reverse()
    for r in dist.batch_isend_irecv(ops):
        r.wait()
    return recv


class _RingAttention(torch.autograd.Function):
    """K/V blocks travel around the ring; partial results are merged with their log-sum-exp."""

    @staticmethod
    def forward(ctx, q, k, v, group, ranks, scale, causal, window, pos_table=None):  # type: ignore[override]
        cp, me = dist.get_world_size(group), dist.get_rank(group)
        sq, sk = q.shape[2], k.shape[2]
        if pos_table is None:  # global token positions held by every rank of the ring
            pos_table = torch.stack([dual_chunk_positions(sk, cp, r, q.device) if causal
                                     else torch.arange(sk, device=q.device) + r * sk for r in range(cp)])
        qpos = pos_table[me]
        kv = torch.stack([k, v]).contiguous()
        out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        lse = torch.full(q.shape[:3], float("-inf"), dtype=torch.float32, device=q.device)
        for step in range(cp):
            src = (me - step) % cp
            kpos = pos_table[src]
            mask = _mask_for(qpos, kpos, causal, window)
            if mask is None or not bool(mask.all()):
                o_b, lse_b = _block_fwd(q, kv[0], kv[1], scale, mask)
                new = torch.logaddexp(lse, lse_b)
                w0 = torch.nan_to_num(torch.exp(lse - new), nan=0.0)[..., None]
                w1 = torch.nan_to_num(torch.exp(lse_b - new), nan=0.0)[..., None]
                out = out * w0 + o_b * w1
                lse = new
            if step != cp - 1:
                kv = _ring_exchange(kv, group, ranks)
        o = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, o, lse, pos_table)
        ctx.cfg = (group, ranks, scale, causal, window)
        return o

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        q, k, v, o, lse, pos_table = ctx.saved_tensors
        group, ranks, scale, causal, window = ctx.cfg
        cp, me = dist.get_world_size(group), dist.get_rank(group)
        qpos = pos_table[me]
        kv = torch.stack([k, v]).contiguous()
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        for step in range(cp):
            src = (me - step) % cp
            kpos = pos_table[src]
            mask = _mask_for(qpos, kpos, causal, window)
            if mask is None or not bool(mask.all()):
                dq_b, dk_b, dv_b = _block_bwd(do, q, kv[0], kv[1], o, lse, scale, mask)
                dq += dq_b
                dkv[0] += dk_b
                dkv[1] += dv_b
            # gradients travel with their K/V block; after cp hops they are back at the owner
            if cp > 1:
                dkv = _ring_exchange(dkv, group, ranks)
                if step != cp - 1:
                    kv = _ring_exchange(kv, group, ranks)
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None, None, None


class _AllGatherSeq(torch.autograd.Function):
    """All-gather along the sequence dim (2); backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        cp = dist.get_world_size(group)
        xs = [torch.empty_like(x) for _ in range(cp)]
        dist.all_gather(xs, x.contiguous(), group=group)
        return torch.stack(xs, dim=0)  # [cp, b, h, s, d]

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        cp = dist.get_world_size(ctx.group)
        out = torch.empty_like(g[0])
        dist.reduce_scatter(out, [g[i].contiguous() for i in range(cp)], group=ctx.group)
        return out, None


class _SeqToHeads(torch.autograd.Function):
    """Ulysses all-to-all: [b, h, s/cp, d] -> [b, h/cp, s, d] (and back in backward)."""

    @staticmethod
    def forward(ctx, x, group, to_heads):  # type: ignore[override]
        ctx.group, ctx.to_heads = group, to_heads
        return _a2a(x, group, to_heads)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return _a2a(g.contiguous(), ctx.group, not ctx.to_heads), None, None


def _a2a(x, group, to_heads):
    cp = dist.get_world_size(group)
    b, h, s, d = x.shape
    if to_heads:
        inp = x.reshape(b, cp, h // cp, s, d).permute(1, 0, 2, 3, 4).contiguous()  # [cp, b, h/cp, s, d]
        out = torch.empty_like(inp)
        dist.all_to_all_single(out, inp, group=group)
        return out.permute(1, 2, 0, 3, 4).reshape(b, h // cp, cp * s, d)  # sequence chunks in rank order
    inp = x.reshape(b, h, cp, s // cp, d).permute(2, 0, 1, 3, 4).contiguous()  # [cp, b, h, s/cp, d]
    out = torch.empty_like(inp)
    dist.all_to_all_single(out, inp, group=group)
    return out.permute(1, 0, 2, 3, 4).reshape(b, cp * h, s // cp, d)


def attn_forward_func_with_cp(q, k, v, *, cp_group, cp_comm_type: str = "p2p", scale: Optional[float] = None,
                              causal: bool = True, window=None, cp_global_ranks=None, cp_stream=None,
                              qkv_format: str = "bhsd", cu_seqlens=None, max_seqlen=None):
    """Attention over the full sequence from per-rank shards; returns ``[b, h, s_local, d]``
    (``[t_local, h, d]`` for ``qkv_format="thd"``, which takes the local cumulative lengths)."""
    if qkv_format == "thd":
        from .context_parallel_thd import thd_ring_attention

        assert cp_comm_type == "p2p" and cu_seqlens is not None, "packed sequences: ring mode with cu_seqlens"
        return thd_ring_attention(q, k, v, cu_seqlens, cp_group=cp_group, scale=scale, causal=causal,
                                  cp_global_ranks=cp_global_ranks, max_seqlen=max_seqlen)
    from ..ops.attention import attention_ref

    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if cp_comm_type == "a2a+p2p":
        return _hierarchical_cp(q, k, v, cp_group, scale, causal, window)
    cp = dist.get_world_size(cp_group)
    me = dist.get_rank(cp_group)
    if cp == 1:
        return attention_ref(q, k, v, scale=scale, causal=causal, window=window)
    if cp_comm_type == "p2p" and _fused_ring_ok(q, k, v, window):
        return fused_ring_attention(q, k, v, cp_group, scale, causal)
    if cp_comm_type == "p2p":
        return _RingAttention.apply(q, k, v, cp_group, cp_global_ranks, scale, causal, window)
    from ..ops.attention import attention as attn_op

    no_window = window is None or (window[0] < 0 and (window[1] < 0 or (causal and window[1] == 0)))
    if cp_comm_type == "all_gather":
        sq, sk = q.shape[2], k.shape[2]
        kg, vg = _AllGatherSeq.apply(k, cp_group), _AllGatherSeq.apply(v, cp_group)
        if no_window:
            # No s x s mask: with the gathered K/V put back in natural order, each of this rank's two
            # query chunks is an ordinary causal attention (diagonal at the bottom-right corner) over the
            # keys up to its own end, so the attention kernels run as they are.
            if causal:
                half = sk // 2
                order = _natural_order_index(half, cp, q.device)
                kf = torch.cat([kg[i] for i in range(cp)], dim=2).index_select(2, order)
                vf = torch.cat([vg[i] for i in range(cp)], dim=2).index_select(2, order)
                hq_ = sq // 2
                outs = []
                for qc, chunk in ((q[:, :, :hq_], me), (q[:, :, hq_:], 2 * cp - 1 - me)):
                    n = (chunk + 1) * half
                    outs.append(attn_op(qc, kf[:, :, :n], vf[:, :, :n], scale=scale, causal=True, bottom_right=True))
                return torch.cat(outs, dim=2)
            kf = torch.cat([kg[i] for i in range(cp)], dim=2)
            vf = torch.cat([vg[i] for i in range(cp)], dim=2)
            return attn_op(q, kf, vf, scale=scale, causal=False)
        kf = torch.cat([kg[i] for i in range(cp)], dim=2)
        vf = torch.cat([vg[i] for i in range(cp)], dim=2)
        if causal:
            qpos = dual_chunk_positions(sq, cp, me, q.device)
            kpos = torch.cat([dual_chunk_positions(sk, cp, r, q.device) for r in range(cp)])
        else:
            qpos = torch.arange(sq, device=q.device) + me * sq
            kpos = torch.arange(sk * cp, device=q.device)
        mask = _mask_for(qpos, kpos, causal, window)
        return attention_ref(q, kf, vf, scale=scale, attn_mask=mask)
    if cp_comm_type == "a2a":
        assert q.shape[1] % cp == 0 and k.shape[1] % cp == 0, "Ulysses needs heads divisible by the CP size"
        qh, kh, vh = (_SeqToHeads.apply(t, cp_group, True) for t in (q, k, v))
        s_full = qh.shape[2]
        if causal:
            # chunks arrive in rank order (dual-chunk layout of every rank): put the sequence in natural
            # order, run plain causal attention over the head shard, and undo the permutation
            order = _natural_order_index(q.shape[2] // 2, cp, q.device)
            inverse = torch.empty_like(order)
            inverse[order] = torch.arange(order.numel(), device=order.device)
            qn, kn, vn = (t.index_select(2, order) for t in (qh, kh, vh))
            on = attn_op(qn, kn, vn, scale=scale, causal=True, window=None if no_window else window)
            oh = on.index_select(2, inverse)
        else:
            oh = attn_op(qh, kh, vh, scale=scale, causal=False, window=None if no_window else window)
        return _SeqToHeads.apply(oh, cp_group, False)
    raise ValueError(f"unknown cp_comm_type {cp_comm_type}")


def _hierarchical_cp(q, k, v, groups, scale, causal, window):
    """Two-level context parallelism (reference ``context_parallel.py:5020``): Ulysses all-to-all inside the first
    group (the NVLink island), then attention across the second group.  The global context-parallel rank of a
    process is ``p2p_rank * a2a_size + a2a_rank``.

    After the all-to-all a process holds ``1 / a2a_size`` of the heads and the tokens of its whole island.  With
    the causal dual-chunk layout those tokens are ``2 * a2a_size`` half-chunks which, put in the right order, are
    exactly the two contiguous chunks that rank ``p2p_rank`` of a ``p2p_size``-way dual-chunk layout owns.  So the
    second level is ordinary context-parallel attention over the outer group: the keys and values are gathered
    across the islands and every query chunk runs as one causal call of the attention kernels (no s x s mask, no
    fp32 block math)."""
    assert isinstance(groups, (list, tuple)) and len(groups) == 2, "a2a+p2p needs [a2a_group, p2p_group]"
    a2a_group, p2p_group = groups
    A = dist.get_world_size(a2a_group)
    s_l = q.shape[2]
    assert q.shape[1] % A == 0 and k.shape[1] % A == 0, "heads must divide by the all-to-all group size"
    qh, kh, vh = (_SeqToHeads.apply(t, a2a_group, True) for t in (q, k, v))
    if causal and A > 1:
        # island member ra contributed chunk (rp * A + ra) then chunk (2 * A * P - 1 - rp * A - ra): first halves in
        # member order, second halves in reverse member order
        half = s_l // 2
        a = torch.arange(half, device=q.device)
        order = torch.cat([ra * s_l + a for ra in range(A)] + [ra * s_l + half + a for ra in reversed(range(A))])
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel(), device=order.device)
        qh, kh, vh = (t.index_select(2, order) for t in (qh, kh, vh))
    else:
        inverse = None
    oh = attn_forward_func_with_cp(qh, kh, vh, cp_group=p2p_group, cp_comm_type="all_gather", scale=scale,
                                   causal=causal, window=window)
    if inverse is not None:
        oh = oh.index_select(2, inverse)
    return _SeqToHeads.apply(oh, a2a_group, False)


# ------------------------------------------------------------------------------------------------
# Fused ring attention on CUDA: the attention kernel reads the peers' K/V over NVLink itself
# ------------------------------------------------------------------------------------------------
class FusedRingAttention:
    """Workspace of context-parallel attention whose K/V exchange is part of the attention kernel.

    Every rank publishes its K/V shard in symmetric memory; the tcgen05 attention kernels
    (``csrc/attn``) then read each peer's shard directly through TMA descriptors on the peer
    address (plain, non-multicast loads), so no K/V tensor is ever staged or sent.  Partial
    results are merged with their log-sum-exp.  In the backward each rank leaves its dK/dV
    contribution for every owner in symmetric memory and the owner sums them with peer loads
    (``csrc/comm/peer_reduce.cu``).  (Reference: ``context_parallel.py:1356`` ring of NCCL
    send/recv around cuDNN attention calls.)
    """

    def __init__(self, group, b: int, hk: int, s_local: int, d: int, dtype):
        from ..ops import _ext
        from .comm_gemm import SymmetricBuffer

        self.group, self.cp, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.shape = (b, hk, s_local, d)
        self.dtype = dtype
        es = torch.empty(0, dtype=dtype).element_size()
        self.shard_bytes = b * hk * s_local * d * es
        total = 2 * self.shard_bytes + self.cp * 2 * self.shard_bytes + 4 * 256 + 8192
        self.buf = SymmetricBuffer(total, group)
        t, self.kv_ptrs = self.buf.carve(2 * self.shard_bytes)
        self.kv = t.view(dtype).reshape(2, b, hk, s_local, d)
        self.kv_off = self.kv_ptrs[self.rank] - self.buf.ptrs[self.rank]
        t, self.dkv_ptrs = self.buf.carve(self.cp * 2 * self.shard_bytes)
        self.dkv = t.view(dtype).reshape(self.cp, 2, b, hk, s_local, d)
        self.flag_ptrs, self.flag_local = [], []
        for _ in range(4):  # kv published, kv read, dkv published, dkv read
            _, p = self.buf.carve(64 * 4)
            self.flag_ptrs.append(p)
            self.flag_local.append(p[self.rank])
        self.epoch = 0
        self.C = _ext.get()
        self.status = self.C.status(self.kv.device.index)
        self.es = es

    def barrier(self, which: int):
        """All ranks have reached this point of the stream (flags in symmetric memory)."""
        self.epoch += 1
        self.C.ep_signal(self.flag_ptrs[which], self.rank, self.epoch, self.status)
        self.C.ep_wait(self.flag_local[which], self.cp, self.epoch, self.status)

    def peer_kv(self, r: int) -> torch.Tensor:
        """Rank ``r``'s published K/V as a tensor on peer memory (only this library's kernels read it)."""
        if r == self.rank:
            return self.kv
        return self.buf.handle.get_buffer(r, (2,) + self.shape, self.dtype, self.kv_off // self.es)

    def publish(self, k, v):
        self.kv[0].copy_(k)
        self.kv[1].copy_(v)
        self.barrier(0)


def _merge(o_run, lse_run, o, lse, rows: slice):
    lr = lse_run[:, :, rows]
    new = torch.logaddexp(lr, lse)
    w0 = torch.nan_to_num(torch.exp(lr - new), nan=0.0)[..., None]
    w1 = torch.nan_to_num(torch.exp(lse - new), nan=0.0)[..., None]
    o_run[:, :, rows] = o_run[:, :, rows] * w0 + o.float() * w1
    lse_run[:, :, rows] = new


def _ring_plan(cp: int, me: int, causal: bool, s: int):
    """(peer, query rows, key rows, causal flag) of every step."""
    half = s // 2
    plan = []
    for step in range(cp):
        r = (me - step) % cp
        if not causal:
            plan.append((r, slice(0, s), slice(0, s), False))
        elif r == me:
            plan.append((r, slice(0, s), slice(0, s), True))
        elif r < me:
            plan.append((r, slice(0, s), slice(0, half), False))
        else:
            plan.append((r, slice(half, s), slice(0, s), False))
    return plan


class _FusedRingAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ws: FusedRingAttention, scale, causal):  # type: ignore[override]
        from ..ops import flash

        b, hq, s, d = q.shape
        ws.publish(k, v)
        o_run = torch.zeros(b, hq, s, d, dtype=torch.float32, device=q.device)
        lse_run = torch.full((b, hq, s), float("-inf"), dtype=torch.float32, device=q.device)
        for r, qrows, krows, csl in _ring_plan(ws.cp, ws.rank, causal, s):
            kv = ws.peer_kv(r)
            o, lse = flash.flash_forward_lse(q[:, :, qrows], kv[0][:, :, krows], kv[1][:, :, krows], scale, csl)
            _merge(o_run, lse_run, o, lse, qrows)
        ws.barrier(1)  # every rank has finished reading: the shards may be overwritten
        out = o_run.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse_run)
        ctx.ws, ctx.scale, ctx.causal = ws, scale, causal
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        q, k, v, out, lse = ctx.saved_tensors
        ws, causal = ctx.ws, ctx.causal
        C_ = ws.C
        b, hq, s, d = q.shape
        sc = float(ctx.scale) if ctx.scale is not None else d ** -0.5
        dout = dout.contiguous()
        ws.publish(k, v)
        ws.dkv.zero_()
        dq = torch.zeros(b, hq, s, d, dtype=torch.float32, device=q.device)
        for r, qrows, krows, csl in _ring_plan(ws.cp, ws.rank, causal, s):
            kv = ws.peer_kv(r)
            qs, os_, dos = q[:, :, qrows], out[:, :, qrows], dout[:, :, qrows]
            n = qs.shape[2]
            s_pad = (n + 127) // 128 * 128
            lse_s = torch.zeros(b, hq, s_pad, dtype=torch.float32, device=q.device)
            lse_s[:, :, :n] = lse[:, :, qrows]
            delta = torch.empty_like(lse_s)
            dq_s = torch.empty(b, hq, n, d, dtype=q.dtype, device=q.device)
            dk_s, dv_s = ws.dkv[r, 0][:, :, krows], ws.dkv[r, 1][:, :, krows]
            C_.flash_bwd(dos, qs, kv[0][:, :, krows], kv[1][:, :, krows], os_, lse_s, delta, dq_s, dk_s, dv_s, sc, csl,
                         True, ws.status)
            dq[:, :, qrows] += dq_s.float()
        ws.barrier(1)
        ws.barrier(2)  # every rank's partial dK/dV are in place
        dkv = torch.empty((2,) + tuple(k.shape), dtype=k.dtype, device=k.device)
        slot = ws.rank * 2 * ws.shard_bytes
        C_.peer_sum([p + slot for p in ws.dkv_ptrs], dkv)
        ws.barrier(3)  # partial buffers may be reused
        return dq.to(q.dtype), dkv[0], dkv[1], None, None, None


_RING_WS: dict = {}


def fused_ring_attention(q, k, v, cp_group, scale, causal):
    b, hk, s, d = k.shape
    key = (id(cp_group), b, hk, s, d, k.dtype)
    if key not in _RING_WS:
        _RING_WS[key] = FusedRingAttention(cp_group, b, hk, s, d, k.dtype)
    return _FusedRingAttn.apply(q, k, v, _RING_WS[key], scale, causal)


def _fused_ring_ok(q, k, v, window) -> bool:
    from ..ops import _ext
    from ..utils.config import get_config

    if not get_config().fused_context_parallel or not _ext.use_cuda(q):
        return False
    if not hasattr(_ext.get(), "flash_fwd") or not hasattr(_ext.get(), "peer_sum"):
        return False
    no_window = window is None or (window[0] < 0 and window[1] <= 0)
    return (q.dtype in (torch.bfloat16, torch.float16) and q.shape[-1] == 128 and v.shape[-1] == 128
            and q.shape[2] == k.shape[2] and q.shape[2] % 128 == 0 and no_window)
