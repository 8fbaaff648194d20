"""Data-parallel gradient synchronisation overlapped with the backward pass.

Every parameter gets a post-accumulate hook that starts an asynchronous NCCL all-reduce
(average) of its gradient as soon as autograd has produced it, so the reductions of the last
layers run while the earlier layers are still in their backward.  Gradients are reduced in
place: no flat buffers, no copies.  Small gradients are batched until ``min_bytes`` is reached
so that launch latency does not dominate.  ``finish()`` makes the current stream wait for all
outstanding reductions; call it before the optimizer step.
(Reference: the data-parallel reduction is left to Megatron / torch DDP; ``pytorch/distributed.py``
only provides the helpers.)
"""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist


class DataParallelGradSync:
    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, min_bytes: int = 32 << 20,
                 average: bool = True, overlap: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.min_bytes = min_bytes
        self.average = average
        self.overlap = overlap  # False: collect during backward, reduce everything in finish()
        self._pending: List[torch.Tensor] = []
        self._pending_bytes = 0
        self._works: list = []
        self._scale_after: List[torch.Tensor] = []
        self._hooks = []
        self.enabled = self.world > 1
        if self.enabled:
            for p in params:
                if p.requires_grad:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def _on_grad(self, p: torch.nn.Parameter) -> None:
        g = p.grad
        if g is None:
            return
        self._pending.append(g)
        self._pending_bytes += g.numel() * g.element_size()
        if self.overlap and self._pending_bytes >= self.min_bytes:
            self._flush()

    def _flush(self) -> None:
        if not self._pending:
            return
        # NCCL averages in the collective; gloo has no AVG, so CPU tensors are summed and scaled in finish()
        nccl_avg = self.average and self._pending[0].is_cuda
        op = dist.ReduceOp.AVG if nccl_avg else dist.ReduceOp.SUM
        for g in self._pending:
            self._works.append(dist.all_reduce(g, op=op, group=self.group, async_op=True))
        if self.average and not nccl_avg:
            self._scale_after.extend(self._pending)
        self._pending, self._pending_bytes = [], 0

    def finish(self) -> None:
        """Wait (stream-wise) for every reduction started during this backward."""
        if not self.enabled:
            return
        self._flush()
        for w in self._works:
            w.wait()
        self._works = []
        for g in self._scale_after:
            g.div_(self.world)
        self._scale_after = []

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []


class ShardedOptimizerDataParallel:
    """Data parallelism with the optimizer sharded over the ranks (ZeRO stage 1 at parameter granularity).

    Every parameter has one owner rank (largest-first greedy assignment, so the owners hold about the
    same number of elements).  During the backward pass each finished gradient is reduced to its owner
    (asynchronously, overlapped with the rest of the backward) instead of all-reduced; only the owner
    keeps optimizer state and updates the parameter; afterwards the owners broadcast the new values.
    Bytes on the wire equal those of the all-reduce it replaces, but the optimizer step and its state
    (fp32 master weights and both moments: 12 of the 16 bytes per parameter) shrink by the group size.

    Usage::

        zero = ShardedOptimizerDataParallel(model.parameters(), group)
        opt = te.FusedAdam(zero.owned_parameters(), master_weights=True, ...)
        ...
        loss.backward(); zero.finish_grads(); opt.step(); zero.sync_parameters()

    (Reference: the reference library provides the building blocks for Megatron's distributed optimizer,
    ``pytorch/tensor/utils.py`` cast_master_weights_to_fp8; the data-parallel reduction itself is the
    framework's.)
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, average: bool = True,
                 overlap: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.average = average
        self.overlap = overlap
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        load = [0] * self.world
        self.owner = {}
        for p in sorted(self.params, key=lambda t: -t.numel()):
            r = min(range(self.world), key=lambda i: load[i])
            self.owner[id(p)] = r
            load[r] += p.numel()
        self._works: list = []
        self._late: List[torch.nn.Parameter] = []
        self._scale_after: List[torch.Tensor] = []
        self._hooks = []
        if self.world > 1:
            for p in self.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def owned_parameters(self) -> List[torch.nn.Parameter]:
        return [p for p in self.params if self.owner[id(p)] == self.rank]

    def _reduce(self, p: torch.nn.Parameter) -> None:
        g = p.grad
        nccl_avg = self.average and g.is_cuda
        op = dist.ReduceOp.AVG if nccl_avg else dist.ReduceOp.SUM
        self._works.append(dist.reduce(g, dst=self._global(self.owner[id(p)]), op=op, group=self.group,
                                       async_op=True))
        if self.average and not nccl_avg and self.owner[id(p)] == self.rank:
            self._scale_after.append(g)

    def _on_grad(self, p: torch.nn.Parameter) -> None:
        if p.grad is None:
            return
        if self.overlap:
            self._reduce(p)
        else:
            self._late.append(p)

    def finish_grads(self) -> None:
        """Wait (stream-wise) for the reductions; gradients of parameters owned elsewhere are dropped."""
        if self.world == 1:
            return
        for p in self._late:
            self._reduce(p)
        self._late = []
        for w in self._works:
            w.wait()
        self._works = []
        for g in self._scale_after:
            g.div_(self.world)
        self._scale_after = []
        for p in self.params:
            if self.owner[id(p)] != self.rank:
                p.grad = None

    def sync_parameters(self) -> None:
        """Owners publish the updated parameters (call after ``optimizer.step()``)."""
        if self.world == 1:
            return
        works = [dist.broadcast(p.data, src=self._global(self.owner[id(p)]), group=self.group, async_op=True)
                 for p in self.params]
        for w in works:
            w.wait()
        from ..modules.base import bump_weights_epoch

        bump_weights_epoch()  # cached quantized weights of the non-owners are stale now

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
