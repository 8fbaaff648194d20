"""FP8 block-scaled tensors (1x128 vectors or 128x128 squares, fp32 scales).

Reference: ``pytorch/tensor/float8_blockwise_tensor.py:28-258``.  On Blackwell the reference converts
these to MXFP8 before the GEMM (``pytorch/csrc/extensions/gemm.cpp:312-323``).  Here the quantize
kernel (``csrc/quant/blockwise.cu``) writes, next to the compact fp32 scales, the same power-of-two
scales as UE8M0 bytes in the tensor core's 128x4-tile layout (each 128-block scale repeated for its
four 32-element sub-blocks), so the block-scaled tcgen05 GEMM multiplies these tensors exactly and
with no conversion pass.  With fp32 (non power-of-two) scales the GEMM operands are dequantized.
"""
from __future__ import annotations

from typing import Iterable

import torch

from ..ops.ref import quant as Q
from .base import QuantizedTensor, QuantizedTensorStorage, Quantizer, pin_payload


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
        # UE8M0 copies of the scales in the GEMM layout (set by the CUDA quantizer for power-of-two scales)
        self._rowwise_mx_scale = None
        self._columnwise_mx_scale = None
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
            self._rowwise_data = self._rowwise_scale_inv = self._rowwise_mx_scale = None
        if columnwise_usage is False:
            self._columnwise_data = self._columnwise_scale_inv = self._columnwise_mx_scale = None

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
        ts = [self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv,
              self._rowwise_mx_scale, self._columnwise_mx_scale]
        self._rowwise_data = self._rowwise_scale_inv = self._columnwise_data = self._columnwise_scale_inv = None
        self._rowwise_mx_scale = self._columnwise_mx_scale = None
        return ts, self

    def restore_from_saved(self, tensors):
        (self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv,
         self._rowwise_mx_scale, self._columnwise_mx_scale) = tensors[:6]
        return tensors[6:]


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

    def is_requantization_safe(self) -> bool:
        return True

    def is_quantizable(self, inp) -> bool:
        return inp.dim() >= 2

    def get_scale_shape(self, shape, columnwise: bool):
        """Shape of the fp32 block scales of a tensor of ``shape``: one per 1 x 128 block (``block_scaling_dim=1``)
        or per 128 x 128 block (2).  The column-wise copy is stored transposed, so its scales are those of a
        ``[last dim, rows]`` matrix."""
        shape = tuple(shape)
        C = shape[-1]
        R = 1
        for d in shape[:-1]:
            R *= d
        if columnwise:
            R, C = C, R
        outer = (R + 127) // 128 if self.block_scaling_dim == 2 else R
        return (outer, (C + 127) // 128)

    def _parts_cuda(self, x2d, rowwise, columnwise):
        """One kernel: both copies, compact fp32 scales and (power-of-two scales) GEMM-layout UE8M0 scales."""
        from ..ops import _ext
        from ..ops.ref.quant import round_up

        x2d = x2d if x2d.stride(-1) == 1 else x2d.contiguous()
        R, C = x2d.shape
        dev, two_d, pow2 = x2d.device, self.block_scaling_dim == 2, bool(self.force_pow_2_scales)
        rkt, ckt = (C + 127) // 128, (R + 127) // 128
        rd = rs = rmx = cd = cs = cmx = None
        if rowwise:
            rd = torch.empty(R, C, dtype=torch.uint8, device=dev)
            rs = torch.empty((round_up(R, 128) // 128 if two_d else R), rkt, dtype=torch.float32, device=dev)
            if pow2 and C % 32 == 0:
                rmx = torch.zeros(round_up(R, 128) * rkt * 4, dtype=torch.uint8, device=dev)
        if columnwise:
            cd = torch.empty(C, R, dtype=torch.uint8, device=dev)
            cs = torch.empty((round_up(C, 128) // 128 if two_d else C), ckt, dtype=torch.float32, device=dev)
            if pow2 and R % 32 == 0:
                cmx = torch.zeros(round_up(C, 128) * ckt * 4, dtype=torch.uint8, device=dev)
        _ext.get().quantize_block128(x2d, 2 if two_d else 1, self.dtype == torch.float8_e5m2, pow2,
                                     float(self.amax_epsilon), rd, rs, rmx, cd, cs, cmx)
        return rd, rs, cd, cs, rmx, cmx

    def _parts(self, x2d, rowwise, columnwise):
        from ..ops import _ext

        if _ext.use_cuda(x2d) and x2d.dtype in (torch.bfloat16, torch.float16, torch.float32):
            return self._parts_cuda(x2d, rowwise, columnwise)
        return self._parts_ref(x2d, rowwise, columnwise) + (None, None)

    def _parts_ref(self, x2d, rowwise, columnwise):
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

    def _wrap(self, rd, rs, cd, cs, shape, hp_dtype, requires_grad=False, rmx=None, cmx=None):
        kw = dict(rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd, columnwise_scale_inv=cs,
                  fp8_dtype=self.dtype, is_2D_scaled=self.block_scaling_dim == 2, quantizer=self, shape=shape,
                  dtype=hp_dtype)
        out = Float8BlockwiseQTensorStorage(**kw) if self.internal else \
            Float8BlockwiseQTensor(requires_grad=requires_grad, **kw)
        out._rowwise_mx_scale, out._columnwise_mx_scale = rmx, cmx
        return out

    def quantize_impl(self, tensor, dtype=None):
        shape = tuple(tensor.shape)
        rd, rs, cd, cs, rmx, cmx = self._parts(tensor.reshape(-1, shape[-1]), self.rowwise_usage,
                                               self.columnwise_usage)
        if rd is not None:
            rd = rd.reshape(shape)
        return self._wrap(rd, rs, cd, cs, shape, dtype or tensor.dtype, rmx=rmx, cmx=cmx)

    def update_quantized(self, src, dst, *, noop_flag=None):
        shape = tuple(dst._shape)
        rd, rs, cd, cs, rmx, cmx = self._parts(src.reshape(-1, shape[-1]), dst._rowwise_data is not None,
                                               dst._columnwise_data is not None)
        if rd is not None:
            dst._rowwise_data.copy_(rd.reshape(shape))
            dst._rowwise_scale_inv.copy_(rs)
            dst._rowwise_mx_scale = rmx if dst._rowwise_mx_scale is None or rmx is None else dst._rowwise_mx_scale.copy_(rmx)
        if cd is not None:
            dst._columnwise_data.copy_(cd)
            dst._columnwise_scale_inv.copy_(cs)
            dst._columnwise_mx_scale = cmx if dst._columnwise_mx_scale is None or cmx is None \
                else dst._columnwise_mx_scale.copy_(cmx)
        return dst

    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False,
                   pin_memory: bool = False):
        x = torch.zeros(tuple(shape), dtype=dtype, device=device)
        was, self.internal = self.internal, False
        try:
            out = self.quantize_impl(x)
        finally:
            self.internal = was
        out.requires_grad_(requires_grad)
        return pin_payload(out) if pin_memory else out
