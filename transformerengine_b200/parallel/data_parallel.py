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
