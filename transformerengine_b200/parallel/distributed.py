"""Collective helpers for tensor / sequence parallel modules, RNG-state tracking and
activation recompute (reference: ``pytorch/distributed.py:241-2257``).

Everything here is plain ``torch.distributed`` (NCCL on GPUs, gloo on CPU) and is
the baseline transport; the fused compute+collective kernels live in
``parallel/comm_gemm.py``.
"""
from __future__ import annotations

import contextlib
from typing import Any, Callable, Dict, Optional, Tuple

import torch
import torch.distributed as dist


def get_world_size(group=None) -> int:
    if not dist.is_available() or not dist.is_initialized():
        return 1
    return dist.get_world_size(group=group)


def get_rank(group=None) -> int:
    if not dist.is_available() or not dist.is_initialized():
        return 0
    return dist.get_rank(group=group)


def gather_along_first_dim(x: torch.Tensor, group, async_op: bool = False):
    """All-gather shards along dim 0.  Returns (tensor, handle or None)."""
    ws = get_world_size(group)
    if ws == 1:
        return x, None
    x = x.contiguous()
    out = torch.empty((x.shape[0] * ws,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    h = dist.all_gather_into_tensor(out, x, group=group, async_op=async_op)
    return out, h


def reduce_scatter_along_first_dim(x: torch.Tensor, group, async_op: bool = False):
    """Sum over ranks, keep this rank's slice of dim 0.  Returns (tensor, handle or None)."""
    ws = get_world_size(group)
    if ws == 1:
        return x, None
    x = x.contiguous()
    assert x.shape[0] % ws == 0, "first dim must divide by the group size"
    out = torch.empty((x.shape[0] // ws,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    h = dist.reduce_scatter_tensor(out, x, group=group, async_op=async_op)
    return out, h


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        return gather_along_first_dim(x, group)[0]

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return reduce_scatter_along_first_dim(g, ctx.group)[0], None


def gather_rows_with_grad(x: torch.Tensor, group) -> torch.Tensor:
    """All-gather along dim 0 whose backward reduce-scatters the gradient (sequence-parallel activations)."""
    return x if get_world_size(group) == 1 else _GatherRows.apply(x, group)


def allreduce(x: torch.Tensor, group, async_op: bool = False):
    if get_world_size(group) == 1:
        return x, None
    h = dist.all_reduce(x, group=group, async_op=async_op)
    return x, h


def allreduce_sequence_parallel_grads(model_or_params, group, *, average: bool = False) -> int:
    """Sum, over the tensor-parallel group, the gradients of every parameter marked ``sequence_parallel``.

    Under sequence parallelism the norm weights (and the biases added after a row-parallel layer) are
    replicated, but each rank sees only its slice of the sequence, so each rank holds a partial
    gradient.  Without this reduction the replicas drift apart.  One flat all-reduce per dtype; call it
    after ``backward()`` and before the optimizer step.  Returns the number of gradients reduced."""
    if get_world_size(group) == 1:
        return 0
    params = model_or_params.parameters() if isinstance(model_or_params, torch.nn.Module) else model_or_params
    by_dtype: Dict[torch.dtype, list] = {}
    for p in params:
        if getattr(p, "sequence_parallel", False) and p.grad is not None:
            by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
    n = 0
    for grads in by_dtype.values():
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=group)
        if average:
            flat.div_(get_world_size(group))
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
        n += len(grads)
    return n


def gather_mxfp8_along_first_dim(q, group):
    """All-gather an MXFP8 tensor sharded on its row dim without dequantizing.

    Rowwise data/scales concatenate along rows; the transposed columnwise copy
    ``[C, R/ws]`` concatenates along its second dim.  Needs the local row count to
    be a multiple of 128 so that whole scale tiles move.
    """
    from ..tensor.mxfp8 import MXFP8TensorStorage
    from ..ops.ref.quant import round_up

    ws = get_world_size(group)
    if ws == 1:
        return q
    R, C = q._rows_cols()
    assert R % 128 == 0, "quantized all-gather needs a multiple of 128 local rows"
    rd = rs = cd = cs = None
    if q._rowwise_data is not None:
        rd, _ = gather_along_first_dim(q._rowwise_data.reshape(R, C), group)
        rs, _ = gather_along_first_dim(q._rowwise_scale_inv, group)
    if q._columnwise_data is not None:
        g, _ = gather_along_first_dim(q._columnwise_data.reshape(1, C, R), group)  # [ws, C, R]
        cd = g.permute(1, 0, 2).reshape(C, ws * R).contiguous()
        kt = round_up(R // 32, 4) // 4
        ct = round_up(C, 128) // 128
        s, _ = gather_along_first_dim(q._columnwise_scale_inv.reshape(1, ct, kt, 512), group)  # [ws, ct, kt, 512]
        cs = s.permute(1, 0, 2, 3).reshape(-1).contiguous()
    shape = (R * ws, C)
    return MXFP8TensorStorage(rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd, columnwise_scale_inv=cs,
                              fp8_dtype=q._fp8_dtype, quantizer=q._quantizer, shape=shape, dtype=q._dtype)


def _gather_cols(t2d: torch.Tensor, group) -> torch.Tensor:
    """All-gather ``[A, B]`` pieces into ``[A, world * B]`` (piece r at columns ``[r * B, (r + 1) * B)``)."""
    ws = get_world_size(group)
    g, _ = gather_along_first_dim(t2d.reshape(1, *t2d.shape), group)     # [ws, A, B]
    return g.permute(1, 0, 2).reshape(t2d.shape[0], ws * t2d.shape[1]).contiguous()


def gather_float8_along_first_dim(q, group):
    """All-gather a per-tensor-scaled FP8 tensor sharded on its rows: one byte per value crosses the wire.
    Every rank must have quantized with the SAME scale (delayed scaling with the amax reduced over a group that
    contains ``group``, or current scaling with the amax reduced over ``group``)."""
    from ..tensor.float8 import Float8TensorStorage

    ws = get_world_size(group)
    if ws == 1:
        return q
    R, C = q._rows_cols()
    data = tr = None
    if q._data is not None:
        data, _ = gather_along_first_dim(q._data.reshape(R, C).view(torch.uint8), group)
        data = data.view(q._data.dtype)
    if q._transpose is not None:
        tr = _gather_cols(q._transpose.reshape(C, R).view(torch.uint8), group).view(q._transpose.dtype)
    return Float8TensorStorage(data=data, fp8_scale_inv=q._scale_inv, fp8_dtype=q._fp8_dtype, data_transpose=tr,
                               quantizer=q._quantizer, shape=(R * ws, C), dtype=q._dtype)


def gather_nvfp4_along_first_dim(q, group):
    """All-gather an NVFP4 tensor sharded on its rows without dequantizing (half a byte per value plus one scale
    byte per 16).  The tensor-wide amaxes must already agree on all ranks (``with_amax_reduction`` over ``group``);
    the local row count must be a multiple of 128 so that whole scale tiles move."""
    from ..tensor.nvfp4 import NVFP4TensorStorage
    from ..ops.ref.quant import round_up

    ws = get_world_size(group)
    if ws == 1:
        return q
    R, C = q._rows_cols()
    assert R % 128 == 0, "quantized all-gather needs a multiple of 128 local rows"
    rd = rs = cd = cs = None
    if q._rowwise_data is not None:
        rd, _ = gather_along_first_dim(q._rowwise_data.reshape(R, C // 2), group)
        rs, _ = gather_along_first_dim(q._rowwise_scale_inv.reshape(-1), group)
    if q._columnwise_data is not None:
        cd = _gather_cols(q._columnwise_data.reshape(C, R // 2), group)
        kt = round_up(R // 16, 4) // 4           # k-tiles (4 scales each) per 128-row tile of the [C, R/16] scale matrix
        ct = round_up(C, 128) // 128
        s, _ = gather_along_first_dim(q._columnwise_scale_inv.reshape(1, ct, kt, 512), group)   # [ws, ct, kt, 512]
        cs = s.permute(1, 0, 2, 3).reshape(-1).contiguous()
    return NVFP4TensorStorage(rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd, columnwise_scale_inv=cs,
                              amax_rowwise=q._amax_rowwise, amax_columnwise=q._amax_columnwise, fp4_dtype=q._fp4_dtype,
                              quantizer=q._quantizer, shape=(R * ws, C), dtype=q._dtype,
                              columnwise_rht=q._columnwise_rht)


def gather_blockwise_along_first_dim(q, group):
    """All-gather a block-scaled FP8 tensor (1 x 128 or 128 x 128 blocks) sharded on its rows without dequantizing;
    the local row count must be a multiple of 128 (whole blocks of the column-wise copy)."""
    from ..tensor.blockwise import Float8BlockwiseQTensorStorage

    ws = get_world_size(group)
    if ws == 1:
        return q
    R, C = q._rows_cols()
    assert R % 128 == 0, "quantized all-gather needs a multiple of 128 local rows"
    rd = rs = cd = cs = None
    if q._rowwise_data is not None:
        rd, _ = gather_along_first_dim(q._rowwise_data.reshape(R, C).view(torch.uint8), group)
        rd = rd.view(q._rowwise_data.dtype)
        rs, _ = gather_along_first_dim(q._rowwise_scale_inv, group)          # [R or R/128, C/128]: rows stack
    if q._columnwise_data is not None:
        cd = _gather_cols(q._columnwise_data.reshape(C, R).view(torch.uint8), group).view(q._columnwise_data.dtype)
        cs = _gather_cols(q._columnwise_scale_inv, group)                      # [C or C/128, R/128]: columns stack
    out = Float8BlockwiseQTensorStorage(rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd,
                                        columnwise_scale_inv=cs, fp8_dtype=q._fp8_dtype, is_2D_scaled=q._is_2D_scaled,
                                        quantizer=q._quantizer, shape=(R * ws, C), dtype=q._dtype)
    return out


def gather_quantized_along_first_dim(q, group):
    """All-gather any quantized tensor sharded on its rows in its quantized form (reference:
    ``pytorch/distributed.py`` ``gather_along_first_dim`` with a quantizer)."""
    from ..tensor.blockwise import Float8BlockwiseQTensorStorage
    from ..tensor.float8 import Float8TensorStorage
    from ..tensor.mxfp8 import MXFP8TensorStorage
    from ..tensor.nvfp4 import NVFP4TensorStorage

    if isinstance(q, MXFP8TensorStorage):
        return gather_mxfp8_along_first_dim(q, group)
    if isinstance(q, Float8TensorStorage):
        return gather_float8_along_first_dim(q, group)
    if isinstance(q, NVFP4TensorStorage):
        return gather_nvfp4_along_first_dim(q, group)
    if isinstance(q, Float8BlockwiseQTensorStorage):
        return gather_blockwise_along_first_dim(q, group)
    raise TypeError(f"no quantized all-gather for {type(q).__name__}")


# --------------------------------------------------------------------------- RNG tracker
# every state that any CudaRNGStatesTracker has registered, by name: CUDA-graph capture code walks this registry to
# register the generators it must keep in step (reference: pytorch/distributed.py, _ALL_ACTIVE_RNG_STATES)
_ALL_ACTIVE_RNG_STATES: Dict[str, torch.Tensor] = {}


def get_all_rng_states() -> Dict[str, torch.Tensor]:
    return _ALL_ACTIVE_RNG_STATES


def set_all_rng_states(states: Dict[str, torch.Tensor]) -> None:
    global _ALL_ACTIVE_RNG_STATES
    _ALL_ACTIVE_RNG_STATES = states


class CudaRNGStatesTracker:
    """Named RNG states so that tensor-parallel ranks can draw the same or different
    random numbers on demand (dropout inside vs outside TP regions)."""

    def __init__(self) -> None:
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_ = set()

    def reset(self) -> None:
        self.states_, self.seeds_ = {}, set()

    def get_states(self) -> Dict[str, torch.Tensor]:
        return dict(self.states_)

    def set_states(self, states: Dict[str, torch.Tensor]) -> None:
        self.states_ = states
        _ALL_ACTIVE_RNG_STATES.update(states)

    @staticmethod
    def _get_state():
        return torch.cuda.get_rng_state() if torch.cuda.is_available() else torch.get_rng_state()

    @staticmethod
    def _set_state(s):
        if torch.cuda.is_available():
            torch.cuda.set_rng_state(s)
        else:
            torch.set_rng_state(s)

    def add(self, name: str, seed: int) -> None:
        if seed in self.seeds_:
            raise RuntimeError(f"seed {seed} already exists")
        if name in self.states_:
            raise RuntimeError(f"cuda rng state {name} already exists")
        self.seeds_.add(seed)
        orig = self._get_state()
        if torch.cuda.is_available():
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states_[name] = self._get_state()
        _ALL_ACTIVE_RNG_STATES[name] = self.states_[name]
        self._set_state(orig)

    @contextlib.contextmanager
    def fork(self, name: str = "model-parallel-rng"):
        if name not in self.states_:
            raise KeyError(f"cuda rng state {name} is not added")
        orig = self._get_state()
        self._set_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = self._get_state()
            _ALL_ACTIVE_RNG_STATES[name] = self.states_[name]
            self._set_state(orig)


# --------------------------------------------------------------------------- activation recompute
_IN_RECOMPUTE = [False]
_IN_CHECKPOINT_FORWARD = [0]
_USE_REENTRANT = [True]      # flavour of the checkpoint in flight (or of the latest one)
_RECOMPUTE_RESTORE: list = []


def is_in_recompute() -> bool:
    """True while a checkpointed region is being run again in the backward pass."""
    return _IN_RECOMPUTE[0]


def in_checkpoint_forward() -> bool:
    """True during the first (activation-discarding) run of a checkpointed region.  Modules with
    delayed-scaling state stash their forward scales then, because the recompute must quantize with
    the same scales although the amax history has moved on in between
    (reference: ``copy_forward_fp8_meta_tensors_for_recompute``, ``pytorch/module/base.py:1601-1649``)."""
    return _IN_CHECKPOINT_FORWARD[0] > 0


def add_recompute_restore(fn: Callable) -> None:
    """Run ``fn`` once the current recompute forward has finished (puts live quantization state back)."""
    _RECOMPUTE_RESTORE.append(fn)


def _run_recompute_restores() -> None:
    todo = list(_RECOMPUTE_RESTORE)
    _RECOMPUTE_RESTORE.clear()
    for fn in reversed(todo):
        fn()


def _consume_first_module_flag() -> None:
    """A checkpointed block has run the forward of its modules without autograd, so none of them took
    the 'first quantized module' token; take it here so that only the first block's recompute owns the
    backward amax reduction."""
    from ..quantization import FP8GlobalStateManager

    if FP8GlobalStateManager.is_fp8_enabled():
        FP8GlobalStateManager.IS_FIRST_FP8_MODULE = False


class _CheckpointFunction(torch.autograd.Function):
    """Re-entrant activation recompute: keep only the inputs, re-run the forward in backward
    under the same RNG state and the same quantization region."""

    @staticmethod
    def forward(ctx, run_function, rng_tracker_fn, kwargs, *args):  # type: ignore[override]
        from ..quantization import FP8GlobalStateManager

        ctx.run_function = run_function
        ctx.kwargs = kwargs
        ctx.rng_tracker_fn = rng_tracker_fn
        ctx.cpu_rng = torch.get_rng_state()
        ctx.cuda_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        ctx.tracker_states = rng_tracker_fn().get_states() if rng_tracker_fn is not None else None
        ctx.autocast_state = FP8GlobalStateManager.get_autocast_state()
        ctx.torch_autocast = torch.is_autocast_enabled()
        _IN_CHECKPOINT_FORWARD[0] += 1
        try:
            with torch.no_grad():
                out = run_function(*args, **kwargs)
        finally:
            _IN_CHECKPOINT_FORWARD[0] -= 1
        _consume_first_module_flag()
        ctx.tensor_idx = [i for i, a in enumerate(args) if torch.is_tensor(a)]
        ctx.others = [None if torch.is_tensor(a) else a for a in args]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        return out

    @staticmethod
    def backward(ctx, *grads):  # type: ignore[override]
        from ..quantization import FP8GlobalStateManager

        saved = list(ctx.saved_tensors)
        args = list(ctx.others)
        for i, t in zip(ctx.tensor_idx, saved):
            args[i] = t.detach().requires_grad_(t.requires_grad)
        cpu_rng = torch.get_rng_state()
        cuda_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        tracker_now = ctx.rng_tracker_fn().get_states() if ctx.rng_tracker_fn is not None else None
        torch.set_rng_state(ctx.cpu_rng)
        if ctx.cuda_rng is not None:
            torch.cuda.set_rng_state(ctx.cuda_rng)
        if ctx.tracker_states is not None:
            ctx.rng_tracker_fn().set_states(ctx.tracker_states)
        cur_state = FP8GlobalStateManager.get_autocast_state()
        FP8GlobalStateManager.set_autocast_state(ctx.autocast_state)
        _IN_RECOMPUTE[0] = True
        try:
            with torch.enable_grad():
                out = ctx.run_function(*args, **ctx.kwargs)
        finally:
            _IN_RECOMPUTE[0] = False
            _run_recompute_restores()
            FP8GlobalStateManager.set_autocast_state(cur_state)
            torch.set_rng_state(cpu_rng)
            if cuda_rng is not None:
                torch.cuda.set_rng_state(cuda_rng)
            if tracker_now is not None:
                ctx.rng_tracker_fn().set_states(tracker_now)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        res = [None, None, None]
        for a in args:
            res.append(a.grad if torch.is_tensor(a) else None)
        return tuple(res)


def checkpoint(function: Callable, *args, distribute_saved_activations: bool = False,
               get_rng_state_tracker: Optional[Callable] = None, tp_group=None, use_reentrant: bool = True,
               **kwargs):
    """Recompute ``function`` in the backward pass instead of storing its activations."""
    if distribute_saved_activations:
        raise NotImplementedError("distribute_saved_activations: saved inputs are kept whole on every rank "
                                  "(use sequence parallelism to shard them)")
    _USE_REENTRANT[0] = bool(use_reentrant)
    if not use_reentrant:
        from torch.utils.checkpoint import checkpoint as torch_ckpt
        from ..quantization import FP8GlobalStateManager

        st = FP8GlobalStateManager.get_autocast_state()

        def ctx_fn():
            @contextlib.contextmanager
            def forward_ctx():
                _IN_CHECKPOINT_FORWARD[0] += 1
                try:
                    yield
                finally:
                    _IN_CHECKPOINT_FORWARD[0] -= 1

            @contextlib.contextmanager
            def recompute_ctx():
                cur = FP8GlobalStateManager.get_autocast_state()
                FP8GlobalStateManager.set_autocast_state(st)
                _IN_RECOMPUTE[0] = True
                try:
                    yield
                finally:
                    _IN_RECOMPUTE[0] = False
                    _run_recompute_restores()
                    FP8GlobalStateManager.set_autocast_state(cur)
            return forward_ctx(), recompute_ctx()

        return torch_ckpt(function, *args, use_reentrant=False, context_fn=ctx_fn, **kwargs)
    return _CheckpointFunction.apply(function, get_rng_state_tracker, kwargs, *args)


def set_tensor_model_parallel_attributes(tensor: torch.Tensor, is_parallel: bool, dim: int, stride: int) -> None:
    setattr(tensor, "tensor_model_parallel", is_parallel)
    setattr(tensor, "partition_dim", dim)
    setattr(tensor, "partition_stride", stride)
