"""Master-weight utilities for sharded optimizers (reference: ``pytorch/tensor/utils.py:204,347,
371,466,593,752``): refresh quantized model weights from fp32 master shards and swap a quantized
tensor's raw storage."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .base import QuantizedTensor, QuantizedTensorStorage


def replace_raw_data(tensor: QuantizedTensorStorage, new_raw_data: torch.Tensor) -> None:
    """Make ``tensor`` use ``new_raw_data`` (same shape/dtype) as its row-wise storage, copying the
    old content over (used to move quantized params into a contiguous all-gather buffer)."""
    for attr in ("_data", "_rowwise_data"):
        old = getattr(tensor, attr, None)
        if old is not None:
            assert old.shape == new_raw_data.shape and old.dtype == new_raw_data.dtype
            new_raw_data.copy_(old)
            setattr(tensor, attr, new_raw_data)
            return
    raise ValueError("tensor holds no raw row-wise data")


def _all_reduce_max(t: torch.Tensor, group) -> torch.Tensor:
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t


def _partial_cast_float8(w, m, off, group) -> None:
    """Per-tensor FP8 weight: the amax of the full weight is the MAX of the shards' amaxes (one float per
    weight crosses the group); every rank then casts only ITS shard into its slice of the raw data
    (reference: ``_cast_master_weights_to_fp8_delayed_scaling`` / ``_current_scaling``,
    ``pytorch/tensor/utils.py:371-592``).  The framework all-gathers the raw bytes afterwards."""
    from ..ops.ref import quant as Q
    from .float8 import Float8CurrentScalingQuantizer

    quant = w._quantizer
    dev = w._data.device if w._data is not None else w._transpose.device
    amax = (m.detach().float().abs().max() if m is not None else torch.zeros((), device=dev)).reshape(1).to(dev)
    amax = _all_reduce_max(amax, group)
    fmax = Q.fp8_max(w._fp8_dtype)
    if isinstance(quant, Float8CurrentScalingQuantizer):
        scale = Q.compute_scale_from_amax(amax, fmax, 0, quant.force_pow_2_scales, quant.amax_epsilon)
    else:  # delayed scaling: the scale is given, the amax is recorded for the next update
        scale = quant.scale.reshape(1).float()
        quant.amax.copy_(torch.maximum(quant.amax.reshape(1), amax).reshape(quant.amax.shape))
    if w._data is None:
        w.update_usage(rowwise_usage=True)
    if m is not None:
        q = Q.quantize_fp8_tensor(m.reshape(-1), scale, w._fp8_dtype)
        w._data.view(-1).view(torch.uint8)[off:off + m.numel()] = q.view(torch.uint8)
    w._scale_inv = (1.0 / scale).reshape(w._scale_inv.shape) if w._scale_inv is not None else 1.0 / scale
    w._transpose = None  # rebuilt from the gathered data (post_all_gather_processing)


def _block_amax_flat(m, off, block_of, nblocks, dev):
    """Partial amax per quantization block of a flat shard: amax[b] = max |m[i]| over the shard's elements i
    (at flat position off + i) whose block index is b; zero elsewhere."""
    out = torch.zeros(nblocks, dtype=torch.float32, device=dev)
    if m is not None and m.numel():
        idx = block_of(torch.arange(off, off + m.numel(), device=dev))
        out.scatter_reduce_(0, idx, m.reshape(-1).float().abs().to(dev), reduce="amax", include_self=True)
    return out


def _partial_cast_mxfp8(w, m, off, group) -> None:
    """MXFP8 weight: one amax per 32-element block, for BOTH copies (blocks along a row for the row-wise
    copy, along a column for the column-wise one).  The shards' partial block amaxes are reduced with MAX
    (numel / 32 floats per copy instead of the full fp32 weight), every rank derives all block scales, and
    casts only its shard's elements (reference: ``common/recipe/mxfp8_scaling.cu:27,78`` partial amax / partial
    cast)."""
    from ..ops.ref import quant as Q

    R, C = w._rows_cols()
    dev = (w._rowwise_data if w._rowwise_data is not None else w._columnwise_data).device
    dt = w._fp8_dtype
    fmax = Q.fp8_max(dt)
    n = m.numel() if m is not None else 0
    flat = torch.arange(off, off + n, device=dev)
    # the MXFP8 quantize kernels read 16-bit values (fp32 inputs are rounded to bf16 first): same here, so that
    # the result equals a quantization of the assembled weight bit for bit
    if m is not None:
        m = m.detach().to(torch.bfloat16).float()
    mv = m.reshape(-1).to(dev) if m is not None else None
    if w._rowwise_data is not None:
        assert C % 32 == 0
        nb = R * (C // 32)
        amax = _all_reduce_max(_block_amax_flat(m, off, lambda i: i // 32, nb, dev), group)
        e = Q.float_to_e8m0(amax * (1.0 / fmax))                       # [R * C/32] uint8
        if n:
            rcp = Q.e8m0_rcp(e)[flat // 32]
            q = torch.clamp(mv * rcp, -fmax, fmax).to(dt)
            w._rowwise_data.view(-1).view(torch.uint8)[off:off + n] = q.view(torch.uint8)
        w._rowwise_scale_inv.copy_(Q.swizzle_scales(e.reshape(R, C // 32)).reshape(w._rowwise_scale_inv.shape))
    if w._columnwise_data is not None:
        assert R % 32 == 0
        nb = C * (R // 32)
        # element (r, c) belongs to column block (c, r // 32) of the transposed copy [C, R]
        blk = lambda i: (i % C) * (R // 32) + (i // C) // 32  # noqa: E731
        amax = _all_reduce_max(_block_amax_flat(m, off, blk, nb, dev), group)
        e = Q.float_to_e8m0(amax * (1.0 / fmax))
        if n:
            rcp = Q.e8m0_rcp(e)[blk(flat)]
            q = torch.clamp(mv * rcp, -fmax, fmax).to(dt)
            pos = (flat % C) * R + flat // C                             # position inside the [C, R] copy
            w._columnwise_data.view(-1).view(torch.uint8)[pos] = q.view(torch.uint8)
        w._columnwise_scale_inv.copy_(Q.swizzle_scales(e.reshape(C, R // 32)).reshape(w._columnwise_scale_inv.shape))


def quantize_master_weights(model_weights: Sequence[torch.Tensor], master_weights: Sequence[Optional[torch.Tensor]],
                            start_offsets: Sequence[Optional[int]], group=None, fsdp_shard_model_weights=None,
                            manual_post_all_gather_processing: bool = False) -> None:
    """Re-quantize each model weight from its fp32 master shard.

    ``master_weights[i]`` is this rank's flat shard of weight ``i`` starting at element
    ``start_offsets[i]`` (``None`` when the rank owns nothing of it).  For per-tensor FP8 and MXFP8 weights
    only amaxes cross ``group`` (one float per tensor, or one per 32-element block): every rank casts its
    own shard into its slice of the weight's raw data, and the caller all-gathers the raw bytes (then calls
    :func:`post_all_gather_processing`).  The column-wise MXFP8 copy is written in place as well (scattered
    positions of the transposed copy), so it needs the same all-gather.  Other formats (and plain weights)
    assemble the full fp32 tensor with an all-reduce and quantize it on every rank.
    ``fsdp_shard_model_weights`` / ``manual_post_all_gather_processing`` (FSDP-sharded model weights, deferred
    post-processing) are not implemented and are refused.
    """
    if fsdp_shard_model_weights is not None or manual_post_all_gather_processing:
        raise NotImplementedError("quantize_master_weights: FSDP-sharded model weights and manual post-all-gather "
                                  "processing are not implemented")
    from .float8 import Float8TensorStorage
    from .mxfp8 import MXFP8TensorStorage

    for w, m, off in zip(model_weights, master_weights, start_offsets):
        off = 0 if off is None else int(off)
        if isinstance(w, Float8TensorStorage) and getattr(w, "_quantizer", None) is not None:
            _partial_cast_float8(w, m, off, group)
            continue
        if isinstance(w, MXFP8TensorStorage):
            _partial_cast_mxfp8(w, m, off, group)
            continue
        full = torch.zeros(w.numel(), dtype=torch.float32, device=w.device)
        if m is not None:
            full[off:off + m.numel()] = m.reshape(-1).float()
            if group is None or dist.get_world_size(group) == 1:
                missing = m.numel() != w.numel()
                if missing:  # keep the part of the weight this rank does not own
                    cur = w.dequantize().float().reshape(-1) if isinstance(w, QuantizedTensorStorage) else \
                        w.detach().float().reshape(-1)
                    mask = torch.ones_like(full, dtype=torch.bool)
                    mask[off:off + m.numel()] = False
                    full[mask] = cur[mask]
        if group is not None and dist.get_world_size(group) > 1:
            dist.all_reduce(full, group=group)
        full = full.reshape(w.shape)
        if isinstance(w, QuantizedTensor):
            w._quantizer.update_quantized(full, w)
        elif isinstance(w, QuantizedTensorStorage):
            w.quantizer.update_quantized(full, w) if hasattr(w, "quantizer") else None
        else:
            w.data.copy_(full.to(w.dtype))


cast_master_weights_to_fp8 = quantize_master_weights  # older name of the same entry point


def post_all_gather_processing(model_weights: Sequence[torch.Tensor]) -> None:
    """After an all-gather of row-wise quantized data, rebuild the column-wise copies."""
    for w in model_weights:
        if isinstance(w, QuantizedTensorStorage) and hasattr(w, "update_usage"):
            w.update_usage(rowwise_usage=True, columnwise_usage=True)


def clear_columnwise_cache(tensor: QuantizedTensorStorage) -> None:
    """Drop the column-wise copy of a quantized tensor that keeps its row-wise bytes (a parameter gathered by FSDP2
    builds that copy on demand, and FSDP cannot free what it did not allocate)."""
    usages = tensor.get_usages() if hasattr(tensor, "get_usages") else {}
    if usages.get("rowwise") and usages.get("columnwise"):
        tensor.update_usage(columnwise_usage=False)


def is_custom(x=None) -> bool:
    """Whether a quantizer / quantized tensor comes from a user recipe (``custom`` attribute); plain tensors do not."""
    if x is None or (isinstance(x, torch.Tensor) and not isinstance(x, QuantizedTensorStorage)):
        return False
    return bool(getattr(x, "custom", False))
