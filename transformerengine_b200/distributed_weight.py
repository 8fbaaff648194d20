"""Extension point for weights that are sharded by an outer framework (weight / "generalised tensor"
parallelism): the parameter a module holds is a shard, and the object itself knows how to assemble
the full matrix for the GEMMs and how to reduce the full weight gradient back onto the shard.

The library defines only the contract and calls it from ``Linear`` (forward GEMM, backward GEMMs,
weight-gradient hand-off); implementations live with the caller.  An implementer is a
``torch.Tensor`` subclass (it is saved for backward and receives the autograd gradient) that sets
``is_distributed_weight = True`` and provides the methods of :class:`DistributedWeight`.  The
dispatch helpers take one weight or a list (grouped modules: the first entry leads its group) and
pass plain tensors through untouched.
(Reference: ``pytorch/distributed_weight.py:26-117``.)
"""
from __future__ import annotations

from typing import Any, List, Protocol, Sequence, runtime_checkable

import torch

__all__ = ["DistributedWeight", "is_distributed_weight", "materialize_weight_for_forward",
           "materialize_weight_for_backward", "finalize_weight_grads"]


@runtime_checkable
class DistributedWeight(Protocol):
    is_distributed_weight: bool

    def materialize_group_for_forward(self) -> Any:
        """Full weight(s) for the forward GEMM (typically an all-gather of the shards)."""

    def materialize_group_for_backward(self) -> Any:
        """Full weight(s) again for the backward GEMMs (nothing is kept alive in between)."""

    def finalize_group_grads(self, wgrads: Any) -> Any:
        """Take the full weight gradient(s) -- e.g. reduce-scatter into ``main_grad`` -- and return
        what autograd should see as the shard's gradient (a dummy, a shard, or ``None``)."""

    def grad_buffer(self) -> torch.Tensor:
        """Accumulation buffer of this weight's gradient."""


def is_distributed_weight(weight: Any) -> bool:
    flag = bool(getattr(weight, "is_distributed_weight", False))
    if flag and not isinstance(weight, torch.Tensor):
        raise TypeError(f"a distributed weight must be a torch.Tensor subclass, got {type(weight).__name__}")
    return flag


def _as_list(x: Any) -> List[Any]:
    return list(x) if isinstance(x, (list, tuple)) else [x]


def materialize_weight_for_forward(weights: Any) -> List[Any]:
    ws = _as_list(weights)
    if ws and is_distributed_weight(ws[0]):
        return _as_list(ws[0].materialize_group_for_forward())
    return ws


def materialize_weight_for_backward(weights: Any) -> List[Any]:
    ws = _as_list(weights)
    if ws and is_distributed_weight(ws[0]):
        return _as_list(ws[0].materialize_group_for_backward())
    return ws


def finalize_weight_grads(weights: Any, wgrads: Sequence[Any]) -> List[Any]:
    ws = _as_list(weights)
    if ws and is_distributed_weight(ws[0]):
        return _as_list(ws[0].finalize_group_grads(wgrads[0] if len(wgrads) == 1 else list(wgrads)))
    return list(wgrads)
