"""Per-tensor scaled FP8 tensors (delayed and current scaling).

Payload: ``_data`` uint8 ``[..., C]``, ``_scale_inv`` fp32 ``[1]`` and an
optional ``_transpose`` uint8 ``[C, R]`` (the columnwise copy).
Reference behaviour: ``pytorch/tensor/float8_tensor.py:53-1099``.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch

from .. import ops
from ..ops.ref import quant as Q
from .base import QuantizedTensor, QuantizedTensorStorage, Quantizer, pin_payload


class Float8TensorStorage(QuantizedTensorStorage):
    def __init__(self, *, data, fp8_scale_inv, fp8_dtype, data_transpose=None, quantizer=None,
                 shape=None, dtype=torch.float32):
        self._data = data
        self._scale_inv = fp8_scale_inv
        self._fp8_dtype = fp8_dtype
        self._transpose = data_transpose
        self._quantizer = quantizer
        self._dtype = dtype
        if shape is None:
            shape = tuple(data.shape) if data is not None else tuple(reversed(data_transpose.shape))
        self._shape = tuple(shape)

    def get_data_tensors(self):
        return self._data, self._transpose

    def get_usages(self):
        return {"rowwise": self._data is not None, "columnwise": self._transpose is not None}

    def update_usage(self, rowwise_usage=None, columnwise_usage=None):
        if columnwise_usage and self._transpose is None and self._data is not None:
            R, C = self._rows_cols()
            self._transpose = self._data.reshape(R, C).t().contiguous()
        if rowwise_usage and self._data is None and self._transpose is not None:
            self._data = self._transpose.t().contiguous().reshape(self._shape)
        if rowwise_usage is False:
            self._data = None
        if columnwise_usage is False:
            self._transpose = None

    def _dequantize_impl(self, dtype=None):
        dtype = dtype or self._dtype
        if self._data is not None:
            return ops.dequantize_fp8(self._data, self._scale_inv, self._fp8_dtype, dtype).reshape(self._shape)
        R, C = self._rows_cols()
        t = ops.dequantize_fp8(self._transpose, self._scale_inv, self._fp8_dtype, dtype)
        return t.t().contiguous().reshape(self._shape)

    def dequantize(self, *, dtype=None):
        return self._dequantize_impl(dtype)

    def prepare_for_saving(self):
        ts = [self._data, self._transpose, self._scale_inv]
        self._data = self._transpose = self._scale_inv = None
        return ts, self

    def restore_from_saved(self, tensors):
        self._data, self._transpose, self._scale_inv = tensors[:3]
        return tensors[3:]


class Float8Tensor(Float8TensorStorage, QuantizedTensor):
    def __new__(cls, *, shape, dtype, data, fp8_scale_inv, fp8_dtype, data_transpose=None,
                quantizer=None, requires_grad=False, device=None):
        dev = device if device is not None else (data if data is not None else data_transpose).device
        self = QuantizedTensor.__new__(cls, shape=shape, dtype=dtype, requires_grad=requires_grad, device=dev)
        Float8TensorStorage.__init__(self, data=data, fp8_scale_inv=fp8_scale_inv, fp8_dtype=fp8_dtype,
                                     data_transpose=data_transpose, quantizer=quantizer, shape=shape, dtype=dtype)
        return self

    def __init__(self, *a, **k):
        pass

    def dequantize(self, *, dtype=None):
        return QuantizedTensor.dequantize(self, dtype=dtype)

    def _new_like(self, requires_grad=None, clone=False, dtype=None):
        c = (lambda t: t.clone() if (clone and t is not None) else t)
        return Float8Tensor(shape=self._shape, dtype=dtype or self._dtype, data=c(self._data),
                            fp8_scale_inv=c(self._scale_inv), fp8_dtype=self._fp8_dtype,
                            data_transpose=c(self._transpose), quantizer=self._quantizer,
                            requires_grad=self.requires_grad if requires_grad is None else requires_grad)

    def __reduce_ex__(self, protocol):
        return (_make_float8_tensor_in_reduce_ex,
                (self._data, self._fp8_dtype, self._scale_inv, self._dtype, self._shape, self._transpose))

    def remove_caches(self) -> None:
        """Drop the transposed copy (it is rebuilt from the row-wise bytes when a GEMM needs it)."""
        if self._data is not None:
            self._transpose = None

    # ---- structural ops that keep the FP8 payload (what FSDP2 does to a parameter when it shards it: chunk along
    # dim 0, allocate a padded buffer, copy the chunk into a slice of it, flatten).  One scale covers the tensor,
    # so every piece shares the scale tensor of its source.
    def _piece(self, data: torch.Tensor) -> "Float8Tensor":
        return Float8Tensor(shape=tuple(data.shape), dtype=self._dtype, data=data, fp8_scale_inv=self._scale_inv,
                            fp8_dtype=self._fp8_dtype, quantizer=self._quantizer, requires_grad=False)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        aten = torch.ops.aten
        t = args[0] if args else None
        if isinstance(t, Float8Tensor) and t._data is not None:
            data = t._data.reshape(t._shape)
            if func == aten.split.Tensor:
                dim = args[2] if len(args) > 2 else kwargs.get("dim", 0)
                return tuple(t._piece(d) for d in torch.split(data, args[1], dim=dim))
            if func == aten.slice.Tensor:
                return t._piece(aten.slice.Tensor(data, *args[1:], **kwargs))
            if func == aten.narrow.default:
                return t._piece(aten.narrow.default(data, *args[1:], **kwargs))
            if func in (aten.view.default, aten._unsafe_view.default, aten.reshape.default):
                return t._piece(data.view(*args[1:]) if func != aten.reshape.default else data.reshape(*args[1:]))
            if func == aten.as_strided.default:
                size, stride = tuple(args[1]), tuple(args[2])
                offset = args[3] if len(args) > 3 and args[3] is not None else 0
                return t._piece(torch.as_strided(data, size, stride, offset))
            if func == aten.new_zeros.default:
                # zero bytes are zero values in both FP8 formats
                size = tuple(args[1])
                dev = kwargs.get("device") or data.device
                return t._piece(torch.zeros(size, dtype=data.dtype, device=dev))
            if func in (aten.empty_like.default, aten.zeros_like.default):
                return t._piece(torch.zeros_like(data))
            if func == aten.copy_.default and isinstance(args[1], Float8Tensor) and args[1]._data is not None \
                    and args[1]._fp8_dtype == t._fp8_dtype and tuple(args[1]._shape) == tuple(t._shape):
                src = args[1]
                data.copy_(src._data.reshape(src._shape))
                if src._scale_inv is not t._scale_inv:
                    t._scale_inv.copy_(src._scale_inv)
                t._transpose = None
                return t
        return super().__torch_dispatch__(func, types, args, kwargs)

    # ---- FSDP2 extension points (reference: tensor/float8_tensor.py:938-1075): shards travel as raw bytes,
    # the per-tensor scale is identical on all ranks (its amax is reduced over the shard group)
    def fsdp_pre_all_gather(self, mesh=None, orig_size=None, contiguous_orig_stride=None, module=None, mp_policy=None):
        if self._data is None:
            self.update_usage(rowwise_usage=True)
        q = self._quantizer
        if mesh is not None and hasattr(q, "with_amax_reduction") and not q.with_amax_reduction:
            # the gathered tensor has ONE scale: from now on every re-quantization of this shard (the optimizer's
            # write-back) takes its amax over all shards, so that the ranks keep agreeing on that scale
            q.with_amax_reduction, q.amax_reduction_group = True, mesh.get_group(mesh.ndim - 1)
        return (self._data.view(torch.uint8),), (self._scale_inv, self._fp8_dtype, self._dtype, self._quantizer)

    def fsdp_post_all_gather(self, all_gather_outputs, metadata, param_dtype=None, *, out=None):
        (data,) = all_gather_outputs
        scale_inv, fp8_dtype, dtype, quantizer = metadata
        if out is not None:
            out._data, out._transpose, out._scale_inv = data, None, scale_inv
            return None
        full = Float8Tensor(shape=data.shape, dtype=dtype, data=data, fp8_scale_inv=scale_inv, fp8_dtype=fp8_dtype,
                            quantizer=quantizer)
        return full, all_gather_outputs


def _make_float8_tensor_in_reduce_ex(data, fp8_dtype, scale_inv, dtype, shape, data_transpose=None):
    return Float8Tensor(shape=shape, dtype=dtype, data=data, fp8_scale_inv=scale_inv, fp8_dtype=fp8_dtype,
                        data_transpose=data_transpose)


class _Float8QuantizerBase(Quantizer):
    dtype: torch.dtype

    def create_tensor_from_data(self, data: torch.Tensor, fake_dtype: torch.dtype = torch.float32,
                                requires_grad: bool = False, internal: bool = False, scale_inv=None):
        """Wrap existing FP8 bytes (uint8, or a float8 tensor viewed as bytes) as a tensor of this quantizer; the
        decode scale is ``scale_inv``, or the reciprocal of the quantizer's current scale."""
        if data.dtype != torch.uint8:
            data = data.view(torch.uint8)
        if scale_inv is None:
            scale = getattr(self, "scale", None)
            scale_inv = torch.ones(1, dtype=torch.float32, device=data.device) if scale is None \
                else scale.detach().float().reshape(1).reciprocal().to(data.device)
        if internal:
            return Float8TensorStorage(data=data, fp8_scale_inv=scale_inv, fp8_dtype=self.dtype, quantizer=self,
                                       shape=tuple(data.shape), dtype=fake_dtype)
        return Float8Tensor(shape=tuple(data.shape), dtype=fake_dtype, data=data, fp8_scale_inv=scale_inv,
                            fp8_dtype=self.dtype, quantizer=self, requires_grad=requires_grad)

    def _wrap(self, data, tr, scale_inv, shape, hp_dtype, requires_grad=False):
        if self.internal:
            return Float8TensorStorage(data=data, fp8_scale_inv=scale_inv, fp8_dtype=self.dtype,
                                       data_transpose=tr, quantizer=self, shape=shape, dtype=hp_dtype)
        return Float8Tensor(shape=shape, dtype=hp_dtype, data=data, fp8_scale_inv=scale_inv,
                            fp8_dtype=self.dtype, data_transpose=tr, quantizer=self, requires_grad=requires_grad)

    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False,
                   pin_memory: bool = False):
        shape = tuple(shape)
        C = shape[-1]
        R = 1
        for s in shape[:-1]:
            R *= s
        data = torch.empty(shape, dtype=torch.uint8, device=device) if self.rowwise_usage else None
        tr = torch.empty(C, R, dtype=torch.uint8, device=device) if self.columnwise_usage else None
        si = torch.ones(1, dtype=torch.float32, device=device)
        was, self.internal = self.internal, False
        try:
            out = self._wrap(data, tr, si, shape, dtype, requires_grad)
        finally:
            self.internal = was
        return pin_payload(out) if pin_memory else out


class Float8Quantizer(_Float8QuantizerBase):
    """Delayed scaling: the scale is given, the observed amax is recorded.

    ``scale`` and ``amax`` are views into the module's recipe state so that the
    amax-history update sees what was recorded here.
    """

    def __init__(self, scale: torch.Tensor, amax: torch.Tensor, fp8_dtype: torch.dtype, *,
                 rowwise: bool = True, columnwise: bool = True):
        super().__init__(rowwise=rowwise, columnwise=columnwise)
        self.scale, self.amax, self.dtype = scale, amax, fp8_dtype

    def quantize_impl(self, tensor, dtype=None):
        shape = tuple(tensor.shape)
        x2d = tensor.reshape(-1, shape[-1])
        data, tr, scale_inv = ops.quantize_fp8(x2d, self.scale, self.dtype, amax_out=self.amax,
                                               rowwise=self.rowwise_usage, columnwise=self.columnwise_usage)
        if data is not None:
            data = data.reshape(shape)
        return self._wrap(data, tr, scale_inv, shape, dtype or tensor.dtype)

    def update_quantized(self, src, dst, *, noop_flag=None):
        shape = tuple(dst._shape)
        x2d = src.reshape(-1, shape[-1])
        want_row = dst._data is not None or dst._transpose is None
        data, tr, scale_inv = ops.quantize_fp8(x2d, self.scale, self.dtype, amax_out=self.amax,
                                               rowwise=want_row, columnwise=dst._transpose is not None)
        if noop_flag is not None and bool(noop_flag.item()):
            return dst
        if data is not None:
            dst._data = data.reshape(shape) if dst._data is None else dst._data.copy_(data.reshape(shape))
        if tr is not None:
            dst._transpose.copy_(tr)
        if dst._scale_inv is None:
            dst._scale_inv = scale_inv
        else:
            dst._scale_inv.copy_(scale_inv)
        return dst

    def calibrate(self, tensor):
        self.amax.copy_(torch.maximum(self.amax.reshape(1), Q.amax_abs(tensor).to(self.amax.device)).reshape(self.amax.shape))


class Float8CurrentScalingQuantizer(_Float8QuantizerBase):
    """Current scaling: amax of the tensor being cast decides its scale."""

    def __init__(self, fp8_dtype: torch.dtype, device=None, *, rowwise=True, columnwise=True,
                 with_amax_reduction=False, amax_reduction_group=None, force_pow_2_scales=False,
                 amax_epsilon=0.0, use_existing_amax: bool = False, scale: Optional[torch.Tensor] = None,
                 amax: Optional[torch.Tensor] = None):
        super().__init__(rowwise=rowwise, columnwise=columnwise)
        self.dtype = fp8_dtype
        self.with_amax_reduction = with_amax_reduction
        self.amax_reduction_group = amax_reduction_group
        self.force_pow_2_scales = force_pow_2_scales
        self.amax_epsilon = amax_epsilon
        # use_existing_amax: the caller (a fused producer kernel, say) has already written the tensor's amax into
        # ``amax``; the quantizer then skips its own reduction pass.  ``scale`` / ``amax`` (fp32 [1]), when given,
        # receive the values used by the latest quantization.
        self.use_existing_amax = use_existing_amax
        self.scale, self.amax = scale, amax
        if use_existing_amax and amax is None:
            raise ValueError("use_existing_amax needs the amax tensor")

    def is_requantization_safe(self) -> bool:
        return True

    def _scale_for(self, tensor):
        if self.use_existing_amax:
            amax = self.amax.detach().float().reshape(-1)[:1].clone().to(tensor.device)
        else:
            amax = ops.amax(tensor)
        if self.with_amax_reduction and self.amax_reduction_group is not None:
            torch.distributed.all_reduce(amax, op=torch.distributed.ReduceOp.MAX, group=self.amax_reduction_group)
        scale = Q.compute_scale_from_amax(amax, Q.fp8_max(self.dtype), 0, self.force_pow_2_scales, self.amax_epsilon)
        if self.amax is not None and not self.use_existing_amax:
            self.amax.copy_(amax.reshape(self.amax.shape))
        if self.scale is not None:
            self.scale.copy_(scale.reshape(self.scale.shape))
        return scale

    def quantize_impl(self, tensor, dtype=None):
        shape = tuple(tensor.shape)
        scale = self._scale_for(tensor)
        data, tr, scale_inv = ops.quantize_fp8(tensor.reshape(-1, shape[-1]), scale, self.dtype,
                                               rowwise=self.rowwise_usage, columnwise=self.columnwise_usage)
        if data is not None:
            data = data.reshape(shape)
        return self._wrap(data, tr, scale_inv, shape, dtype or tensor.dtype)

    def update_quantized(self, src, dst, *, noop_flag=None):
        shape = tuple(dst._shape)
        scale = self._scale_for(src)
        data, tr, scale_inv = ops.quantize_fp8(src.reshape(-1, shape[-1]), scale, self.dtype,
                                               rowwise=dst._data is not None or dst._transpose is None,
                                               columnwise=dst._transpose is not None)
        if data is not None:
            dst._data = data.reshape(shape) if dst._data is None else dst._data.copy_(data.reshape(shape))
        if tr is not None:
            dst._transpose.copy_(tr)
        if dst._scale_inv is None:
            dst._scale_inv = scale_inv
        else:
            dst._scale_inv.copy_(scale_inv)
        return dst
