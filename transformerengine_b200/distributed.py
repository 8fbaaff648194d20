"""Distributed helpers under the reference's module name (``pytorch/distributed.py``): the implementations live in
``parallel/distributed.py``; this module adds the small query / chunking helpers that training frameworks import."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .constants import dist_group_type  # noqa: F401
from .parallel.distributed import (CudaRNGStatesTracker, allreduce, allreduce_sequence_parallel_grads,  # noqa: F401
                                   checkpoint, gather_along_first_dim, gather_quantized_along_first_dim,
                                   in_checkpoint_forward, is_in_recompute, reduce_scatter_along_first_dim,
                                   set_tensor_model_parallel_attributes)
from .parallel.distributed import get_rank as get_distributed_rank  # noqa: F401
from .parallel.distributed import get_world_size as get_distributed_world_size  # noqa: F401


def is_fp8_activation_recompute_enabled() -> bool:
    """True while the forward pass of a checkpointed region runs (quantization state is recorded for the recompute)."""
    return in_checkpoint_forward()


def in_fp8_activation_recompute_phase() -> bool:
    """True while a checkpointed region is being recomputed in the backward pass."""
    return is_in_recompute()


def split_tensor_into_1d_equal_chunks(tensor: torch.Tensor, tp_group, new_buffer: bool = False) -> torch.Tensor:
    """This rank's contiguous 1-D chunk of ``tensor`` (flattened, split evenly over ``tp_group``)."""
    ws, rank = get_distributed_world_size(tp_group), get_distributed_rank(tp_group)
    flat = tensor.reshape(-1)
    n = flat.numel() // ws
    chunk = flat[rank * n:(rank + 1) * n]
    return chunk.clone() if new_buffer else chunk


def gather_split_1d_tensor(tensor: torch.Tensor, tp_group) -> torch.Tensor:
    """Inverse of :func:`split_tensor_into_1d_equal_chunks`: all-gather the 1-D chunks."""
    ws = get_distributed_world_size(tp_group)
    if ws == 1:
        return tensor.reshape(-1)
    out = torch.empty(ws * tensor.numel(), dtype=tensor.dtype, device=tensor.device)
    dist.all_gather_into_tensor(out, tensor.reshape(-1).contiguous(), group=tp_group)
    return out


def symmetric_all_reduce(inp: torch.Tensor, tp_group=None, async_op: bool = False, all_reduce_type: str = "one_shot"):
    """All-reduce of an activation.  The reference picks a symmetric-memory algorithm by ``all_reduce_type``; here
    the fused GEMM + all-reduce kernel (``te.initialize_ub``) covers the row-parallel layer, and a bare tensor goes
    through NCCL (which uses in-switch reduction on NVSwitch systems by itself)."""
    return allreduce(inp, tp_group, async_op=async_op)


def prepare_te_modules_for_fsdp(fsdp_root: torch.nn.Module) -> None:
    """Tag every module of this library under ``fsdp_root`` so that it knows its parameters are sharded by FSDP
    (activations saved for backward then keep no reference to full parameters)."""
    from .modules.base import TransformerEngineBaseModule

    for m in fsdp_root.modules():
        if isinstance(m, TransformerEngineBaseModule):
            m.fsdp_wrapped = True
            m.fsdp_group = getattr(fsdp_root, "process_group", None)
