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
