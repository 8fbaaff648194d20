"""Fused optimizers under the reference's package name (``pytorch/optimizers``); the implementations live in
``optim/``.

The multi-tensor operations are exported in the calling convention that ``multi_tensor_applier`` uses in the
reference, ``op(chunk_size, noop_flag, tensor_lists, *args)``::

    norm, _ = multi_tensor_applier(multi_tensor_l2norm, overflow_buf, [grads], False)
    multi_tensor_applier(multi_tensor_scale, overflow_buf, [grads, grads], clip_coeff)

(``chunk_size`` is accepted and ignored: the kernels pick their own chunking.)"""
import torch

from .. import ops as _ops
from ..optim import *  # noqa: F401,F403
from ..optim import FusedAdam, FusedSGD, multi_tensor_applier  # noqa: F401


class MultiTensorApply:
    """Callable with a fixed chunk size (``MultiTensorApply(2048 * 32)(op, noop, lists, *args)``)."""

    available = True

    def __init__(self, chunk_size: int):
        self.chunk_size = chunk_size

    def __call__(self, op, noop_flag_buffer, tensor_lists, *args):
        return op(self.chunk_size, noop_flag_buffer, tensor_lists, *args)


def multi_tensor_scale(chunk_size, noop_flag, tensor_lists, scale):
    """``tensor_lists = [src, dst]``: ``dst = src * scale``; ``noop_flag`` is set to 1 when a source holds inf / nan."""
    _ops.multi_tensor_scale(tensor_lists, float(scale), noop_flag)


def multi_tensor_scale_tensor(chunk_size, noop_flag, tensor_lists, scale):
    """As ``multi_tensor_scale`` with the scale in a device tensor (no host read on a GPU: the products are formed
    with tensor operations)."""
    src, dst = tensor_lists
    s = scale.reshape(()).float()
    for a, b in zip(src, dst):
        if noop_flag is not None:
            noop_flag.copy_(torch.maximum(noop_flag, (~torch.isfinite(a).all()).to(noop_flag.dtype).reshape(noop_flag.shape)))
        b.copy_((a.float() * s).to(b.dtype))


def multi_tensor_l2norm(chunk_size, noop_flag, tensor_lists, per_tensor: bool = False):
    """``tensor_lists = [tensors]``: returns ``(global L2 norm [1], per-tensor norms or an empty tensor)``."""
    total, each = _ops.multi_tensor_l2norm(list(tensor_lists[0]), bool(per_tensor))
    return total, (each if each is not None else total.new_zeros(0))


def multi_tensor_unscale_l2norm(chunk_size, noop_flag, tensor_lists, inv_scale, per_tensor: bool = False):
    """L2 norm of ``tensors * inv_scale`` (gradients that still carry a loss scale)."""
    total, each = multi_tensor_l2norm(chunk_size, noop_flag, tensor_lists, per_tensor)
    inv = inv_scale.reshape(()).float() if isinstance(inv_scale, torch.Tensor) else float(inv_scale)
    return total * inv, (each * inv if each.numel() else each)


__all__ = ["FusedAdam", "FusedSGD", "MultiTensorApply", "multi_tensor_applier", "multi_tensor_scale",
           "multi_tensor_scale_tensor", "multi_tensor_l2norm", "multi_tensor_unscale_l2norm"]
