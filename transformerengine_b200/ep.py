"""Expert-parallel dispatch / combine under the reference's module name (``pytorch/ep.py``).

Two call forms share ``ep_dispatch`` / ``ep_combine``:

* this library's own: ``ep_dispatch(x, probs, routing_map, group, local_experts, align)`` ->
  ``(tokens, probs, m_splits, state)`` and ``ep_combine(expert_out, state)`` (``parallel/expert_parallel.py``; the
  fused peer-memory kernels have their own entry points there);
* the reference's buffer API: ``ep_bootstrap(group, ...)`` once, one ``EpBuffer`` per micro-batch in flight,
  ``ep_dispatch(buffer, tokens, topk_idx, topk_weights)`` -> ``(recv_tokens, recv_topk_weights,
  tokens_per_expert)`` and ``ep_combine(buffer, expert_out)`` -> ``[num_local_tokens, hidden]``.  Received rows
  are grouped by LOCAL expert (each expert's rows padded up to ``alignment``, the padding rows are zero with weight
  zero); ``tokens_per_expert`` holds the padded counts, i.e. the ``m_splits`` of a ``GroupedLinear``.  Without a
  ``recv_capacity_per_rank`` the outputs are sized per step ("eager": the counts are read on the host); with one,
  the outputs always have that many rows (the tail is zero) and a step that receives more raises, or drops the
  excess rows of the last experts with ``drop_on_overflow``.

The buffer API here runs on the all-to-all transport (NCCL or gloo); MXFP8 payloads on the wire
(``dispatch_fwd_quant_recipe`` / ``combine_bwd_quant_recipe``), zero-copy symmetric-memory IO and CUDA-graph capture
of the exchange are not implemented in it and are refused.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .parallel import expert_parallel as _impl
from .parallel.expert_parallel import *  # noqa: F401,F403

_EP = {"group": None, "cfg": None}


def ep_bootstrap(ep_group, num_experts: int, max_tokens_per_rank: int, hidden_dim: int, num_topk: int,
                 recv_capacity_per_rank: Optional[int] = None, max_num_sms: int = 0, zero_copy: bool = False,
                 drop_on_overflow: bool = False, max_token_dtype: torch.dtype = torch.bfloat16) -> None:
    """Register the expert-parallel group and its sizes.  Call once per process, before creating buffers."""
    if zero_copy:
        raise NotImplementedError("zero_copy: the buffer API copies through the all-to-all transport; the peer-memory "
                                  "path is parallel.expert_parallel.fused_ep_dispatch / fused_ep_combine")
    if drop_on_overflow and recv_capacity_per_rank is None:
        raise ValueError("drop_on_overflow requires recv_capacity_per_rank")
    world = dist.get_world_size(ep_group)
    if num_experts % world:
        raise ValueError(f"num_experts ({num_experts}) must divide by the group size ({world})")
    _EP["group"] = ep_group
    _EP["cfg"] = dict(num_experts=int(num_experts), max_tokens_per_rank=int(max_tokens_per_rank),
                      hidden_dim=int(hidden_dim), num_topk=int(num_topk),
                      recv_capacity_per_rank=None if recv_capacity_per_rank is None else int(recv_capacity_per_rank),
                      drop_on_overflow=bool(drop_on_overflow), max_token_dtype=max_token_dtype)


def is_ep_bootstrapped() -> bool:
    return _EP["group"] is not None


def ep_finalize() -> None:
    """Forget the group (call before destroying it); idempotent."""
    _EP["group"], _EP["cfg"] = None, None


def is_symm_backed(t: torch.Tensor) -> bool:
    """Whether ``t`` lives in symmetric memory of the expert-parallel group.  The buffer API never allocates there."""
    try:
        from torch.distributed import _symmetric_memory as symm
        if hasattr(symm, "is_symm_mem_tensor"):
            return bool(symm.is_symm_mem_tensor(t))
    except Exception:  # noqa: BLE001
        pass
    return False


class EpBuffer:
    """Per-micro-batch state of one dispatch / combine pair."""

    def __init__(self, top_k: int, max_tokens_per_rank: int, hidden_dim: int, num_local_experts: int,
                 recv_capacity_per_rank: Optional[int] = None, alignment: int = 0,
                 payload_dtype: torch.dtype = torch.bfloat16, device=None, dispatch_fwd_quant_recipe=None,
                 combine_bwd_quant_recipe=None) -> None:
        if not is_ep_bootstrapped():
            raise RuntimeError("EpBuffer requires ep_bootstrap() to be called first.")
        alignment = int(alignment)
        if alignment > 1 and alignment & (alignment - 1):
            raise ValueError(f"alignment must be 0, 1, or a power of two (got {alignment}).")
        if dispatch_fwd_quant_recipe is not None or combine_bwd_quant_recipe is not None:
            raise NotImplementedError("quantized payloads on the wire are not implemented: tokens travel in their own "
                                      "dtype and the expert layers quantize what they receive")
        cfg = _EP["cfg"]
        self.eager = cfg["recv_capacity_per_rank"] is None
        if not self.eager and recv_capacity_per_rank is None:
            recv_capacity_per_rank = cfg["recv_capacity_per_rank"]
        if self.eager and recv_capacity_per_rank is not None:
            raise ValueError("the group was bootstrapped without recv_capacity_per_rank (eager mode): buffers cannot "
                             "have one")
        self.top_k, self.alignment = int(top_k), alignment
        self.max_tokens_per_rank, self.hidden_dim = int(max_tokens_per_rank), int(hidden_dim)
        self.recv_capacity_per_rank = None if recv_capacity_per_rank is None else int(recv_capacity_per_rank)
        self.num_local_experts = int(num_local_experts)
        self.payload_dtype, self.device = payload_dtype, device
        self.zero_copy = False
        self.dispatch_fwd_quant_recipe = self.combine_bwd_quant_recipe = None
        self.tokens_per_expert: Optional[torch.Tensor] = None    # int64 [num_local_experts], padded counts
        self.total_recv_tokens: Optional[torch.Tensor] = None    # int64 [1]
        self._state = None                                        # exchange plan of the latest dispatch
        self._rows = 0


def _dense_routing(buffer: EpBuffer, topk_idx: torch.Tensor, topk_weights: Optional[torch.Tensor]):
    if topk_idx.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"topk_idx must be int32 or int64, got {topk_idx.dtype}")
    E = _EP["cfg"]["num_experts"]
    idx = topk_idx.reshape(-1, topk_idx.shape[-1]).long()
    rmap = torch.zeros(idx.shape[0], E, dtype=torch.bool, device=idx.device).scatter_(1, idx, True)
    probs = None
    if topk_weights is not None:
        probs = torch.zeros(idx.shape[0], E, dtype=topk_weights.dtype, device=idx.device).scatter(
            1, idx, topk_weights.reshape(idx.shape))
    return probs, rmap


def ep_prepare(buffer: EpBuffer, topk_idx: torch.Tensor) -> torch.Tensor:
    """Exchange the routing counts: returns (and stores) ``tokens_per_expert`` (int64 ``[num_local_experts]``,
    padded to the buffer's alignment) and fills ``buffer.total_recv_tokens``."""
    group = _EP["group"]
    _, rmap = _dense_routing(buffer, topk_idx, None)
    world, me = dist.get_world_size(group), dist.get_rank(group)
    counts = rmap.sum(0).to(torch.int64)
    allc = torch.empty(world * counts.numel(), dtype=torch.int64, device=counts.device)
    dist.all_gather_into_tensor(allc, counts.contiguous(), group=group)
    L = buffer.num_local_experts
    mine = allc.reshape(world, -1)[:, me * L:(me + 1) * L].sum(0)
    a = max(buffer.alignment, 1)
    buffer.tokens_per_expert = (mine + a - 1) // a * a
    buffer.total_recv_tokens = buffer.tokens_per_expert.sum().reshape(1)
    return buffer.tokens_per_expert


def _fit_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    if t.shape[0] > rows:
        return t[:rows]
    pad = torch.zeros((rows - t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    return torch.cat([t, pad])


def ep_dispatch(*args, **kwargs):
    """See the module docstring for the two call forms."""
    if not args or not isinstance(args[0], EpBuffer):
        return _impl.ep_dispatch(*args, **kwargs)
    return _buffer_dispatch(*args, **kwargs)


def _buffer_dispatch(buffer: EpBuffer, tokens: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, *,
                     recv_tokens: Optional[torch.Tensor] = None, recv_topk_weights: Optional[torch.Tensor] = None):
    if topk_weights.dtype is not torch.float32:
        raise TypeError(f"topk_weights must be float32; got dtype={topk_weights.dtype}. Cast with "
                        "topk_weights.float() before calling.")
    if buffer.eager and (recv_tokens is not None or recv_topk_weights is not None):
        raise ValueError("eager mode sizes the recv outputs from the per-step recv-token total and cannot use "
                         "caller-supplied recv_tokens / recv_topk_weights")
    x = tokens.reshape(-1, tokens.shape[-1])
    probs, rmap = _dense_routing(buffer, topk_idx, topk_weights)
    xs, ps, m_splits, state = _impl.ep_dispatch(x, probs, rmap, _EP["group"], buffer.num_local_experts,
                                                max(buffer.alignment, 1))
    buffer._state, buffer._rows = state, xs.shape[0]
    buffer.tokens_per_expert = torch.tensor(m_splits, dtype=torch.int64, device=x.device)
    buffer.total_recv_tokens = buffer.tokens_per_expert.sum().reshape(1)
    cap = buffer.recv_capacity_per_rank
    if cap is not None:
        if xs.shape[0] > cap:
            if not _EP["cfg"]["drop_on_overflow"]:
                raise RuntimeError(f"this rank received {xs.shape[0]} rows, more than recv_capacity_per_rank={cap}")
            # dropped rows belong to the last experts; their counts shrink accordingly
            kept = torch.clamp(cap - (buffer.tokens_per_expert.cumsum(0) - buffer.tokens_per_expert), min=0)
            buffer.tokens_per_expert = torch.minimum(buffer.tokens_per_expert, kept)
        xs, ps = _fit_rows(xs, cap), _fit_rows(ps, cap)
        if recv_tokens is not None:
            recv_tokens.copy_(xs.detach())
        if recv_topk_weights is not None:
            recv_topk_weights.copy_(ps.detach())
    return xs, ps, buffer.tokens_per_expert


def ep_combine(*args, **kwargs):
    """See the module docstring for the two call forms."""
    if not args or not isinstance(args[0], EpBuffer):
        return _impl.ep_combine(*args, **kwargs)
    return _buffer_combine(*args, **kwargs)


def _buffer_combine(buffer: EpBuffer, expert_out: torch.Tensor, *, num_local_tokens: Optional[int] = None,
                    grad_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Send the expert outputs (the caller has applied the routing weights) back and sum them per source token."""
    if buffer._state is None:
        raise RuntimeError("ep_combine needs the buffer of the matching ep_dispatch")
    if buffer.eager and grad_out is not None:
        raise ValueError("eager mode sizes the combine grad target per step and cannot use a caller-supplied grad_out")
    out = _impl.ep_combine(_fit_rows(expert_out, buffer._rows), buffer._state)
    n = out.shape[0] if num_local_tokens is None else int(num_local_tokens)
    return _fit_rows(out, n)
