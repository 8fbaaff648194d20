"""Expert-parallel token exchange: dispatch tokens to the ranks that own their experts and
combine the expert outputs back (reference API ``pytorch/ep.py:830-953`` over NCCL-EP; here
``all_to_all_single`` over NCCL / gloo is the baseline transport, and the permutation, padding
and chunk re-ordering are this library's own ops).

Layout produced by :func:`ep_dispatch`: rows grouped by LOCAL expert, each slab padded to
``align`` rows, ready for ``GroupedLinear``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..moe.permutation import _dest_rows_from_mask


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):  # type: ignore[override]
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        out = torch.empty((sum(ctx.in_splits),) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


@dataclass
class EPState:
    group: object
    dest: torch.Tensor          # [T, E] row of each (token, expert) pair in the local expert-major buffer
    send_splits: List[int]      # rows sent to every rank
    recv_splits: List[int]      # rows received from every rank
    recv_counts: torch.Tensor   # [ep, local_experts] rows per (source rank, local expert)
    order: torch.Tensor         # gather index: padded expert-major row -> received row (or -1 for padding)
    num_tokens: int
    n_recv: int


def ep_dispatch(x: torch.Tensor, probs: torch.Tensor, routing_map: torch.Tensor, group, local_experts: int,
                align: int = 1) -> Tuple[torch.Tensor, torch.Tensor, List[int], EPState]:
    """Returns (tokens for the local experts [sum(m_splits), H], their routing probs, m_splits, state)."""
    ep = dist.get_world_size(group)
    T, H = x.shape
    E = routing_map.shape[1]
    dest, counts, _ = _dest_rows_from_mask(routing_map, 1)  # expert-major: experts of rank 0 first
    valid = dest >= 0
    tok = torch.arange(T, device=x.device)[:, None].expand_as(dest)[valid]
    rows = dest[valid]
    n_send = int(counts.sum().item())
    send = torch.zeros(n_send, H, dtype=x.dtype, device=x.device).index_put((rows,), x[tok])
    send_p = torch.zeros(n_send, dtype=probs.dtype, device=x.device).index_put((rows,), probs[valid])
    # counts exchange: every rank learns how many rows each source sends to each of its experts
    flat_counts = torch.empty(ep * E, dtype=counts.dtype, device=x.device)
    dist.all_gather_into_tensor(flat_counts, counts.contiguous(), group=group)
    all_counts = flat_counts.reshape(ep, E)
    me = dist.get_rank(group)
    recv_counts = all_counts[:, me * local_experts:(me + 1) * local_experts]  # [src, local expert]
    send_splits = counts.reshape(ep, local_experts).sum(1).tolist()
    recv_splits = recv_counts.sum(1).tolist()
    recv = _AllToAll.apply(send, recv_splits, send_splits, group)
    recv_p = _AllToAll.apply(send_p, recv_splits, send_splits, group)
    # received order is [src][local expert]; experts want [local expert][src], padded
    rc = recv_counts.t().contiguous()  # [local expert, src]
    per_expert = rc.sum(1)
    padded = (per_expert + align - 1) // align * align
    m_splits = [int(v) for v in padded.tolist()]
    starts_src_major = torch.zeros(ep * local_experts + 1, dtype=torch.int64, device=x.device)
    starts_src_major[1:] = recv_counts.reshape(-1).cumsum(0)
    order = torch.full((sum(m_splits),), -1, dtype=torch.int64, device=x.device)
    pos = 0
    rc_l = rc.tolist()
    for e in range(local_experts):
        p = pos
        for s in range(ep):
            n = rc_l[e][s]
            if n:
                st = int(starts_src_major[s * local_experts + e].item())
                order[p:p + n] = torch.arange(st, st + n, device=x.device)
                p += n
        pos += m_splits[e]
    keep = order >= 0
    xs = torch.zeros(len(order), H, dtype=x.dtype, device=x.device)
    ps = torch.zeros(len(order), dtype=probs.dtype, device=x.device)
    if recv.shape[0]:
        xs = xs.index_put((keep.nonzero(as_tuple=True)[0],), recv[order[keep]])
        ps = ps.index_put((keep.nonzero(as_tuple=True)[0],), recv_p[order[keep]])
    state = EPState(group, dest, send_splits, recv_splits, recv_counts, order, T, int(recv.shape[0]))
    return xs, ps, m_splits, state


def ep_combine(expert_out: torch.Tensor, state: EPState) -> torch.Tensor:
    """Send expert outputs back to the ranks that own the tokens and sum the top-k contributions."""
    H = expert_out.shape[1]
    keep = state.order >= 0
    back = torch.zeros(state.n_recv, H, dtype=expert_out.dtype, device=expert_out.device)
    if state.n_recv:
        back = back.index_put((state.order[keep],), expert_out[keep.nonzero(as_tuple=True)[0]])
    ret = _AllToAll.apply(back, state.send_splits, state.recv_splits, state.group)
    dest = state.dest
    valid = dest >= 0
    tok = torch.arange(state.num_tokens, device=expert_out.device)[:, None].expand_as(dest)[valid]
    vals = ret[dest[valid]]
    out = torch.zeros(state.num_tokens, H, dtype=torch.float32, device=expert_out.device)
    return out.index_add(0, tok, vals.float()).to(expert_out.dtype)


# ------------------------------------------------------------------------------------------------
# Fused path: permutation and all-to-all in one kernel over NVLink peer memory
# ------------------------------------------------------------------------------------------------
class FusedExpertParallel:
    """Symmetric-memory workspace and epoch counter of one expert-parallel group.

    ``dispatch`` stores every routed token row straight into the owning rank's expert-major
    buffer (``csrc/comm/moe_a2a.cu: ep_push_kernel``); ``combine`` reads the expert outputs back
    from the owners and sums them per token (``ep_pull_kernel``).  All ranks must call the
    operations in the same order; every call advances a shared epoch that the flags carry.
    """

    def __init__(self, group, local_experts: int, hidden: int, max_tokens: int, dtype=torch.bfloat16,
                 align: int = 128, topk: Optional[int] = None):
        from .comm_gemm import SymmetricBuffer

        self.group, self.L, self.H, self.dtype, self.align = group, local_experts, hidden, dtype, align
        self.ep, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.E = self.ep * self.L
        per_tok = min(topk or self.L, self.L)
        self.cap = self.ep * max_tokens * per_tok + self.L * align
        self.cap = (self.cap + align - 1) // align * align
        es = torch.empty(0, dtype=dtype).element_size()
        row_bytes = hidden * es
        assert row_bytes % 16 == 0
        total = 2 * self.cap * row_bytes + 2 * self.cap * 4 + self.ep * self.E * 4 + 3 * 64 * 4 + 8192
        self.buf = SymmetricBuffer(total, group)
        t, self.recv_ptrs = self.buf.carve(self.cap * row_bytes)
        self.recv = t.view(dtype).reshape(self.cap, hidden)
        t, self.out_ptrs = self.buf.carve(self.cap * row_bytes)
        self.out_buf = t.view(dtype).reshape(self.cap, hidden)
        t, self.recv_probs_ptrs = self.buf.carve(self.cap * 4)
        self.recv_probs = t.view(torch.float32)
        t, self.out_s_ptrs = self.buf.carve(self.cap * 4)
        self.out_s = t.view(torch.float32)
        _, self.counts_ptrs = self.buf.carve(self.ep * self.E * 4)
        self.flag_ptrs = []
        self.flag_local = []
        for _ in range(3):  # counts published, rows pushed, rows ready to be pulled
            t, p = self.buf.carve(64 * 4)
            self.flag_ptrs.append(p)
            self.flag_local.append(p[self.rank])
        dev = self.recv.device
        self.base = torch.zeros(self.E, dtype=torch.int32, device=dev)
        self.splits = torch.zeros(self.L + 1, dtype=torch.int32, device=dev)
        self.seg = torch.zeros(self.L * (self.ep + 1), dtype=torch.int32, device=dev)
        self.counter = torch.zeros(4, dtype=torch.int32, device=dev)
        self.epoch = 0
        self.C = _ext_get()
        self.status = self.C.status(dev.index)

    # ---- primitives -----------------------------------------------------------------------------
    def _push(self, x, within, probs, scale, rowmap, base):
        self.epoch += 1
        self.C.ep_push(x.contiguous(), within, base, scale, probs, self.recv_ptrs,
                       self.recv_probs_ptrs if probs is not None else [], self.flag_ptrs[1], rowmap, self.counter,
                       self.L, self.rank, self.cap, self.epoch, self.status)
        self.C.ep_wait(self.flag_local[1], self.ep, self.epoch, self.status)

    def _publish_and_pull(self, rows, rowmap, T, scalars=None):
        n = rows.shape[0]
        self.out_buf[:n].copy_(rows)
        if scalars is not None:
            self.out_s[:n].copy_(scalars)
        self.epoch += 1
        self.C.ep_signal(self.flag_ptrs[2], self.rank, self.epoch, self.status)
        self.C.ep_wait(self.flag_local[2], self.ep, self.epoch, self.status)
        out = torch.empty(T, self.H, dtype=self.dtype, device=rows.device)
        outs = torch.empty(T, self.E, dtype=torch.float32, device=rows.device) if scalars is not None else None
        self.C.ep_pull(self.out_ptrs, rowmap, None, out, None, None, self.L,
                       self.out_s_ptrs if scalars is not None else [], outs)
        return out, outs

    def _take(self, total: int, seg: List[int], with_probs: bool):
        """Copy the received rows out of the workspace and zero the padding between expert slabs."""
        xs = self.recv[:total].clone()
        ps = self.recv_probs[:total].clone() if with_probs else None
        pos = 0
        for el in range(self.L):
            end = seg[el * (self.ep + 1) + self.ep]
            nxt = seg[(el + 1) * (self.ep + 1)] if el + 1 < self.L else total
            if nxt > end:
                xs[end:nxt] = 0
                if ps is not None:
                    ps[end:nxt] = 0
            pos = nxt
        return xs, ps


def _ext_get():
    from ..ops import _ext

    return _ext.get()


@dataclass
class FusedEPState:
    ctx: "FusedExpertParallel"
    within: torch.Tensor      # [T, E] int32
    rowmap: torch.Tensor      # [T, E] int32
    total: int
    seg: List[int]
    num_tokens: int
    base: Optional[torch.Tensor] = None   # [E] int32 row bases of this routing


class _FusedDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, routing_map, ep: FusedExpertParallel, holder: dict):  # type: ignore[override]
        m = routing_map.bool()
        T = x.shape[0]
        counts = m.sum(0).to(torch.int32)
        # rank of token t among this rank's tokens of expert e: scan along the token axis of the
        # TRANSPOSED mask (a scan over the outer dim of [T, E] is ~300x slower in torch)
        mt = m.t().contiguous()
        within_t = torch.where(mt, mt.cumsum(1, dtype=torch.int32) - 1, torch.full((), -1, dtype=torch.int32, device=x.device))
        within = within_t.t().contiguous()
        ep.epoch += 1
        ep.C.ep_counts(ep.counts_ptrs, ep.flag_ptrs[0], counts, ep.base, ep.splits, ep.seg, ep.L, ep.rank, ep.align,
                       ep.epoch, ep.status)
        rowmap = torch.empty(T, ep.E, dtype=torch.int32, device=x.device)
        pf = probs.float().contiguous()
        base = ep.base.clone()  # later dispatches through the same workspace overwrite ep.base
        ep._push(x, within, pf, None, rowmap, base)
        host = torch.cat([ep.splits, ep.seg]).tolist()  # one synchronising read: split sizes for the grouped GEMM
        splits, seg = host[:ep.L + 1], host[ep.L + 1:]
        total = splits[ep.L]
        xs, ps = ep._take(total, seg, True)
        state = FusedEPState(ep, within, rowmap, total, seg, T, base)
        ctx.state, ctx.pdtype = state, probs.dtype
        ctx.mark_non_differentiable(rowmap)
        ctx.save_for_backward(m)
        holder["state"] = state
        holder["m_splits"] = [int(v) for v in splits[:ep.L]]
        return xs, ps.to(probs.dtype), rowmap

    @staticmethod
    def backward(ctx, g_xs, g_ps, _g_rowmap):  # type: ignore[override]
        st = ctx.state
        (m,) = ctx.saved_tensors
        gp = g_ps.float().contiguous() if g_ps is not None else torch.zeros(st.total, device=g_xs.device)
        gx, gs = st.ctx._publish_and_pull(g_xs.contiguous(), st.rowmap, st.num_tokens, gp)
        gprobs = torch.where(m, gs, torch.zeros((), device=gs.device)).to(ctx.pdtype)
        return gx, gprobs, None, None, None


class _FusedCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, state: FusedEPState):  # type: ignore[override]
        ctx.state = state
        out, _ = state.ctx._publish_and_pull(expert_out.contiguous(), state.rowmap, state.num_tokens)
        return out

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        st = ctx.state
        ep = st.ctx
        scratch = torch.empty_like(st.rowmap)
        ep._push(g.contiguous(), st.within, None, None, scratch, st.base)
        gy, _ = ep._take(st.total, st.seg, False)
        return gy, None


def fused_ep_dispatch(x, probs, routing_map, ep: FusedExpertParallel):
    """Fused counterpart of :func:`ep_dispatch`: returns (tokens, probs, m_splits, state)."""
    holder: dict = {}
    xs, ps, _ = _FusedDispatch.apply(x, probs, routing_map, ep, holder)
    return xs, ps, holder["m_splits"], holder["state"]


def fused_ep_combine(expert_out, state: FusedEPState):
    return _FusedCombine.apply(expert_out, state)


_EP_CONTEXTS: dict = {}


def get_fused_ep(group, local_experts: int, hidden: int, max_tokens: int, dtype, align: int, topk: int):
    key = (id(group), local_experts, hidden, max_tokens, dtype, align, topk)
    if key not in _EP_CONTEXTS:
        _EP_CONTEXTS[key] = FusedExpertParallel(group, local_experts, hidden, max_tokens, dtype, align, topk)
    return _EP_CONTEXTS[key]
