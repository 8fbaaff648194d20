"""FP8 block-scaled tensors (1x128 vectors or 128x128 squares, fp32 scales).

Reference: ``pytorch/tensor/float8_blockwise_tensor.py:28-258``.  On Blackwell
the reference converts these to MXFP8 before the GEMM
(``pytorch/csrc/extensions/gemm.cpp:312-323``); this library dequantizes the
block scales into the MXFP8 kernel the same way when power-of-two scales are
used, and otherwise multiplies in high precision.
"""
from __future__ import annotations

from typing import Iterable

import torch

from ..ops.ref import quant as Q
from .base import QuantizedTensor, QuantizedTensorStorage, Quantizer


class Float8BlockwiseQTensorStorage(QuantizedTensorStorage):
    def __init__(self, *, rowwise_data, rowwise_scale_inv, columnwise_data, columnwise_scale_inv, fp8_dtype,
                 is_2D_scaled, quantizer=None, shape=None, dtype=torch.float32):
        self._rowwise_data = rowwise_data
        self._rowwise_scale_inv = rowwise_scale_inv
        self._columnwise_data = columnwise_data  # transposed [C, R]
        self._columnwise_scale_inv = columnwise_scale_inv
        self._fp8_dtype = fp8_dtype
        self._is_2D_scaled = is_2D_scaled
        self._quantizer = quantizer
        self._dtype = dtype
        if shape is None:
            shape = tuple(rowwise_data.shape) if rowwise_data is not None else tuple(reversed(columnwise_data.shape))
        self._shape = tuple(shape)

    def _dims(self):
        return (128, 128) if self._is_2D_scaled else (1, 128)

    def get_data_tensors(self):
        return self._rowwise_data, self._columnwise_data

    def get_usages(self):
        return {"rowwise": self._rowwise_data is not None, "columnwise": self._columnwise_data is not None}

    def update_usage(self, rowwise_usage=None, columnwise_usage=None):
        if rowwise_usage is False:
            self._rowwise_data = self._rowwise_scale_inv = None
        if columnwise_usage is False:
            self._columnwise_data = self._columnwise_scale_inv = None

    def _dequantize_impl(self, dtype=None):
        dtype = dtype or self._dtype
        R, C = self._rows_cols()
        if self._rowwise_data is not None:
            q = self._rowwise_data.reshape(R, C).view(self._fp8_dtype)
            return Q.dequantize_fp8_blockwise(q, self._rowwise_scale_inv, self._dims(), dtype).reshape(self._shape)
        q = self._columnwise_data.view(self._fp8_dtype)
        out = Q.dequantize_fp8_blockwise(q, self._columnwise_scale_inv, self._dims(), dtype)
        return out.t().contiguous().reshape(self._shape)

    def dequantize(self, *, dtype=None):
        return self._dequantize_impl(dtype)

    def prepare_for_saving(self):
        ts = [self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv]
        self._rowwise_data = self._rowwise_scale_inv = self._columnwise_data = self._columnwise_scale_inv = None
        return ts, self

    def restore_from_saved(self, tensors):
        (self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data,
         self._columnwise_scale_inv) = tensors[:4]
        return tensors[4:]


class Float8BlockwiseQTensor(Float8BlockwiseQTensorStorage, QuantizedTensor):
    def __new__(cls, *, shape, dtype, rowwise_data, rowwise_scale_inv, columnwise_data, columnwise_scale_inv,
                fp8_dtype, is_2D_scaled, quantizer=None, requires_grad=False, device=None):
        dev = device if device is not None else (rowwise_data if rowwise_data is not None else columnwise_data).device
        self = QuantizedTensor.__new__(cls, shape=shape, dtype=dtype, requires_grad=requires_grad, device=dev)
        Float8BlockwiseQTensorStorage.__init__(
            self, rowwise_data=rowwise_data, rowwise_scale_inv=rowwise_scale_inv, columnwise_data=columnwise_data,
            columnwise_scale_inv=columnwise_scale_inv, fp8_dtype=fp8_dtype, is_2D_scaled=is_2D_scaled,
            quantizer=quantizer, shape=shape, dtype=dtype)
        return self

    def __init__(self, *a, **k):
        pass

    def dequantize(self, *, dtype=None):
        return QuantizedTensor.dequantize(self, dtype=dtype)

    def _new_like(self, requires_grad=None, clone=False, dtype=None):
        c = (lambda t: t.clone() if (clone and t is not None) else t)
        return Float8BlockwiseQTensor(
            shape=self._shape, dtype=dtype or self._dtype, rowwise_data=c(self._rowwise_data),
            rowwise_scale_inv=c(self._rowwise_scale_inv), columnwise_data=c(self._columnwise_data),
            columnwise_scale_inv=c(self._columnwise_scale_inv), fp8_dtype=self._fp8_dtype,
            is_2D_scaled=self._is_2D_scaled, quantizer=self._quantizer,
            requires_grad=self.requires_grad if requires_grad is None else requires_grad)

    def __reduce_ex__(self, protocol):
        return (_make_blockwise_in_reduce_ex,
                (self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv,
                 self._fp8_dtype, self._is_2D_scaled, self._dtype, self._shape))


def _make_blockwise_in_reduce_ex(rd, rs, cd, cs, fp8_dtype, is_2d, dtype, shape):
    return Float8BlockwiseQTensor(shape=shape, dtype=dtype, rowwise_data=rd, rowwise_scale_inv=rs,
                                  columnwise_data=cd, columnwise_scale_inv=cs, fp8_dtype=fp8_dtype,
                                  is_2D_scaled=is_2d)


class Float8BlockQuantizer(Quantizer):
    def __init__(self, fp8_dtype=torch.float8_e4m3fn, *, rowwise=True, columnwise=True, amax_epsilon=0.0,
                 force_pow_2_scales=True, block_scaling_dim=1):
        super().__init__(rowwise=rowwise, columnwise=columnwise)
        self.dtype = fp8_dtype
        self.amax_epsilon = amax_epsilon
        self.force_pow_2_scales = force_pow_2_scales
        self.block_scaling_dim = block_scaling_dim

    def _parts(self, x2d, rowwise, columnwise):
        dims = (128, 128) if self.block_scaling_dim == 2 else (1, 128)
        rd = rs = cd = cs = None
        if rowwise:
            q, rs = Q.quantize_fp8_blockwise(x2d, self.dtype, dims, self.force_pow_2_scales, self.amax_epsilon)
            rd = q.view(torch.uint8)
        if columnwise:
            q, cs = Q.quantize_fp8_blockwise(x2d.t().contiguous(), self.dtype, dims, self.force_pow_2_scales,
                                             self.amax_epsilon)
            cd = q.view(torch.uint8)
        return rd, rs, cd, cs

    def _wrap(self, rd, rs, cd, cs, shape, hp_dtype, requires_grad=False):
        kw = dict(rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd, columnwise_scale_inv=cs,
                  fp8_dtype=self.dtype, is_2D_scaled=self.block_scaling_dim == 2, quantizer=self, shape=shape,
                  dtype=hp_dtype)
        if self.internal:
            return Float8BlockwiseQTensorStorage(**kw)
        return Float8BlockwiseQTensor(requires_grad=requires_grad, **kw)

    def quantize_impl(self, tensor, dtype=None):
        shape = tuple(tensor.shape)
        rd, rs, cd, cs = self._parts(tensor.reshape(-1, shape[-1]), self.rowwise_usage, self.columnwise_usage)
        if rd is not None:
            rd = rd.reshape(shape)
        return self._wrap(rd, rs, cd, cs, shape, dtype or tensor.dtype)

    def update_quantized(self, src, dst, *, noop_flag=None):
        shape = tuple(dst._shape)
        rd, rs, cd, cs = self._parts(src.reshape(-1, shape[-1]), dst._rowwise_data is not None,
                                     dst._columnwise_data is not None)
        if rd is not None:
            dst._rowwise_data.copy_(rd.reshape(shape))
            dst._rowwise_scale_inv.copy_(rs)
        if cd is not None:
            dst._columnwise_data.copy_(cd)
            dst._columnwise_scale_inv.copy_(cs)
        return dst

    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False):
        x = torch.zeros(tuple(shape), dtype=dtype, device=device)
        was, self.internal = self.internal, False
        try:
            out = self.quantize_impl(x)
        finally:
            self.internal = was
        out.requires_grad_(requires_grad)
        return out
