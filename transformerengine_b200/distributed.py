"""Distributed helpers under the reference's module name (``pytorch/distributed.py``): the implementations live in
``parallel/distributed.py``; this module adds the small query / chunking helpers that training frameworks import."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .constants import dist_group_type  # noqa: F401
from .parallel.distributed import (CudaRNGStatesTracker, allreduce_sequence_parallel_grads,  # noqa: F401
                                   checkpoint, gather_quantized_along_first_dim,
                                   get_all_rng_states, in_checkpoint_forward, is_in_recompute,
                                   set_all_rng_states, set_tensor_model_parallel_attributes)
from .parallel import distributed as _impl
from .parallel.distributed import get_rank as get_distributed_rank  # noqa: F401
from .parallel.distributed import get_world_size as get_distributed_world_size  # noqa: F401


def gather_along_first_dim(inp, process_group=None, async_op: bool = False, quantizer=None, output_tensor=None,
                           external_coalescing: bool = False, group=None):
    """All-gather along dim 0; returns ``(tensor, handle)``.  With ``quantizer`` (or a quantized ``inp``) the
    QUANTIZED payload travels: the input is quantized first and the result is a quantized tensor of the gathered
    shape (row-wise copy; formats that need it rebuild their column-wise copy from the gathered rows)."""
    from .tensor.base import QuantizedTensorStorage
    g = process_group if process_group is not None else group
    if external_coalescing:
        raise NotImplementedError("external_coalescing: issue the gathers inside torch.distributed's own coalescing "
                                  "manager instead")
    if quantizer is not None or isinstance(inp, QuantizedTensorStorage):
        q = inp if isinstance(inp, QuantizedTensorStorage) else quantizer(inp)
        return gather_quantized_along_first_dim(q, g), None
    out, handle = _impl.gather_along_first_dim(inp, g, async_op=async_op)
    if output_tensor is not None:
        if handle is not None:
            handle.wait()
            handle = None
        output_tensor.copy_(out)
        out = output_tensor
    return out, handle


def reduce_scatter_along_first_dim(inp, tp_group=None, async_op: bool = False, output=None, group=None):
    """Reduce-scatter along dim 0; returns ``(tensor, handle)``."""
    out, handle = _impl.reduce_scatter_along_first_dim(inp, tp_group if tp_group is not None else group,
                                                      async_op=async_op)
    if output is not None:
        if handle is not None:
            handle.wait()
            handle = None
        output.copy_(out)
        out = output
    return out, handle


def allreduce(inp, tp_group=None, async_op: bool = False, group=None):
    """All-reduce (sum); returns ``(tensor, handle)``."""
    return _impl.allreduce(inp, tp_group if tp_group is not None else group, async_op=async_op)


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


def graph_safe_rng_available() -> bool:
    """Whether this PyTorch can register generator states with a CUDA graph (so that captured random draws advance
    between replays)."""
    return (hasattr(torch.cuda.CUDAGraph, "register_generator_state") and hasattr(torch.Generator, "graphsafe_set_state")
            and hasattr(torch.Generator, "graphsafe_get_state") and hasattr(torch.Generator, "clone_state"))


def is_graph_safe_rng_state(state) -> bool:
    return graph_safe_rng_available() and isinstance(state, torch.Generator)


def initialize_affine_weight_gpu(weight: torch.Tensor, init_method, get_rng_state_tracker, partition_dim: int = 0,
                                 stride: int = 1, set_tp_attributes: bool = True) -> None:
    """Initialise a tensor-parallel weight shard under the tracker's model-parallel random stream (every rank
    draws its own values) and tag it with its partitioning."""
    if set_tp_attributes:
        set_tensor_model_parallel_attributes(weight, True, partition_dim, stride)
    if get_rng_state_tracker is None:
        init_method(weight)
        return
    with get_rng_state_tracker().fork():
        init_method(weight)


class activation_recompute_forward:  # noqa: N801  (a context manager with the reference's spelling)
    """Marks the two passes of a checkpointed region for code that drives recomputation itself instead of calling
    ``checkpoint``: ``activation_recompute=True, recompute_phase=False`` around the first (activation-discarding)
    forward, ``recompute_phase=True`` around the second one in the backward pass.  Modules with delayed-scaling
    state stash their forward scales in the first and reuse them in the second."""

    def __init__(self, activation_recompute: bool = False, recompute_phase: bool = False):
        self.activation_recompute, self.recompute_phase = activation_recompute, recompute_phase

    def __enter__(self):
        self._was = (_impl._IN_CHECKPOINT_FORWARD[0], _impl._IN_RECOMPUTE[0])
        if self.activation_recompute and not self.recompute_phase:
            _impl._IN_CHECKPOINT_FORWARD[0] += 1
        if self.activation_recompute and self.recompute_phase:
            _impl._IN_RECOMPUTE[0] = True
        return self

    def __exit__(self, *exc):
        _impl._IN_CHECKPOINT_FORWARD[0], _impl._IN_RECOMPUTE[0] = self._was
        if self.activation_recompute and self.recompute_phase:
            _impl._run_recompute_restores()
        return False

    def __call__(self, fn):
        import functools

        @functools.wraps(fn)
        def wrapped(*a, **k):
            with activation_recompute_forward(self.activation_recompute, self.recompute_phase):
                return fn(*a, **k)
        return wrapped


def get_activation_recompute_contexts():
    """``(forward context, recompute context)`` for a hand-written checkpoint."""
    return activation_recompute_forward(True, False), activation_recompute_forward(True, True)


def use_reentrant_activation_recompute() -> bool:
    """Whether the checkpoint in flight uses the re-entrant autograd function (the default of ``checkpoint``)."""
    return getattr(_impl, "_USE_REENTRANT", [True])[0]


def get_te_classes():
    """Module classes of this library (what ``has_te_modules`` looks for)."""
    from .attention.dot_product_attention import DotProductAttention
    from .attention.multi_head_attention import MultiheadAttention
    from .modules.base import TransformerEngineBaseModule
    from .modules.layernorm_linear import LayerNorm, RMSNorm
    from .transformer import TransformerLayer
    return (LayerNorm, RMSNorm, TransformerEngineBaseModule, DotProductAttention, MultiheadAttention, TransformerLayer)


def has_te_modules(network) -> bool:
    """Whether ``network`` contains modules of this library (anything that is not an ``nn.Module`` counts as yes:
    a bare callable cannot be inspected)."""
    if isinstance(network, torch.nn.Module):
        return any(isinstance(m, get_te_classes()) for m in network.modules())
    return True
