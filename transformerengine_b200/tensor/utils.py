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


def quantize_master_weights(model_weights: Sequence[torch.Tensor], master_weights: Sequence[Optional[torch.Tensor]],
                            start_offsets: Sequence[Optional[int]], group=None, fsdp_shard_model_weights=None,
                            manual_post_all_gather_processing: bool = False) -> None:
    """Re-quantize each model weight from its fp32 master shard.

    ``master_weights[i]`` is this rank's flat shard of weight ``i`` starting at element
    ``start_offsets[i]`` (``None`` when the rank owns nothing of it).  The shards are assembled
    across ``group`` (sum of zero-padded shards), then every rank quantizes the full tensor with
    the weight's own quantizer, so scales agree on all ranks.
    """
    for w, m, off in zip(model_weights, master_weights, start_offsets):
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
