"""MXFP8 tensors: FP8 data with one UE8M0 scale per 32 values.

Payload:
  ``_rowwise_data``      uint8 ``[..., C]``   blocks of 32 along the last dim
  ``_rowwise_scale_inv`` uint8, 128x4-tile swizzled, padded ``[ru(R,128) * ru(C/32,4)]``
  ``_columnwise_data``   uint8 ``[C, R]``     TRANSPOSED; blocks of 32 along R
  ``_columnwise_scale_inv`` uint8 swizzled, padded ``[ru(C,128) * ru(R/32,4)]``

The reference keeps the columnwise copy untransposed
(``pytorch/tensor/mxfp8_tensor.py:139-180``) and lets cuBLASLt read it
MN-major; here the quantize kernel writes it transposed at no extra memory
traffic so that all tcgen05 operands are K-major.  ``to_reference_layout``
converts for checkpoint exchange.
"""
from __future__ import annotations

from typing import Iterable

import torch

from .. import ops
from ..ops.ref import quant as Q
from .base import QuantizedTensor, QuantizedTensorStorage, Quantizer


class MXFP8TensorStorage(QuantizedTensorStorage):
    def __init__(self, *, rowwise_data, rowwise_scale_inv, columnwise_data, columnwise_scale_inv,
                 fp8_dtype, quantizer=None, shape=None, dtype=torch.float32):
        self._rowwise_data = rowwise_data
        self._rowwise_scale_inv = rowwise_scale_inv
        self._columnwise_data = columnwise_data
        self._columnwise_scale_inv = columnwise_scale_inv
        self._fp8_dtype = fp8_dtype
        self._quantizer = quantizer
        self._dtype = dtype
        self._with_gemm_swizzled_scales = True
        if shape is None:
            shape = tuple(rowwise_data.shape) if rowwise_data is not None else tuple(reversed(columnwise_data.shape))
        self._shape = tuple(shape)

    def get_data_tensors(self):
        return self._rowwise_data, self._columnwise_data

    def get_usages(self):
        return {"rowwise": self._rowwise_data is not None, "columnwise": self._columnwise_data is not None}

    def update_usage(self, rowwise_usage=None, columnwise_usage=None):
        # the two copies are different quantizations: a missing one cannot be rebuilt
        if rowwise_usage and self._rowwise_data is None:
            raise RuntimeError("MXFP8 tensor has no rowwise copy")
        if columnwise_usage and self._columnwise_data is None:
            raise RuntimeError("MXFP8 tensor has no columnwise copy")
        if rowwise_usage is False:
            self._rowwise_data = self._rowwise_scale_inv = None
        if columnwise_usage is False:
            self._columnwise_data = self._columnwise_scale_inv = None

    def ensure_columnwise(self) -> None:
        """Build the column-wise copy from the row-wise one when it is missing (a parameter that FSDP2 has just
        gathered carries only the row-wise bytes).  The row-wise values are exact in bf16, so this is a second
        rounding of already rounded values, along the other direction; only dgrad reads the result."""
        if self._columnwise_data is not None or self._rowwise_data is None or len(self._shape) != 2:
            return
        R, C = self._rows_cols()
        if R % 32 or C % 32:
            return
        hp = ops.dequantize_mxfp8(self._rowwise_data.reshape(R, C), self._rowwise_scale_inv, self._fp8_dtype,
                                  torch.bfloat16)
        two_d = bool(getattr(self._quantizer, "with_2d_quantization", False))    # then the rebuilt copy is exact
        _, _, cd, cs = ops.quantize_mxfp8(hp, self._fp8_dtype, rowwise=False, columnwise=True, two_d=two_d)
        self._columnwise_data, self._columnwise_scale_inv = cd, cs

    def _dequantize_impl(self, dtype=None):
        dtype = dtype or self._dtype
        R, C = self._rows_cols()
        if self._rowwise_data is not None:
            out = ops.dequantize_mxfp8(self._rowwise_data.reshape(R, C), self._rowwise_scale_inv,
                                       self._fp8_dtype, dtype)
            return out.reshape(self._shape)
        out = ops.dequantize_mxfp8(self._columnwise_data, self._columnwise_scale_inv, self._fp8_dtype, dtype)
        return out.t().contiguous().reshape(self._shape)

    def dequantize(self, *, dtype=None):
        return self._dequantize_impl(dtype)

    def prepare_for_saving(self):
        ts = [self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv]
        self._rowwise_data = self._rowwise_scale_inv = None
        self._columnwise_data = self._columnwise_scale_inv = None
        return ts, self

    def restore_from_saved(self, tensors):
        (self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data,
         self._columnwise_scale_inv) = tensors[:4]
        return tensors[4:]

    def to_reference_layout(self):
        """(rowwise_data, rowwise_scale [Rp,Kp] compact, columnwise_data [R,C],
        columnwise_scale [ru(R/32,4), ru(C,128)] compact) as the reference stores them."""
        R, C = self._rows_cols()
        rs = cs = cd = None
        if self._rowwise_scale_inv is not None:
            rs = Q.pad_scales(Q.unswizzle_scales(self._rowwise_scale_inv, R, C // 32))
        if self._columnwise_data is not None:
            cd = self._columnwise_data.t().contiguous().reshape(self._shape)
            cs_t = Q.unswizzle_scales(self._columnwise_scale_inv, C, R // 32)  # [C, R/32]
            cs = Q.pad_scales(cs_t.t().contiguous(), 4, 128)
        return self._rowwise_data, rs, cd, cs


class MXFP8Tensor(MXFP8TensorStorage, QuantizedTensor):
    def __new__(cls, *, shape, dtype, rowwise_data, rowwise_scale_inv, columnwise_data, columnwise_scale_inv,
                fp8_dtype, quantizer=None, requires_grad=False, device=None):
        dev = device if device is not None else (rowwise_data if rowwise_data is not None else columnwise_data).device
        self = QuantizedTensor.__new__(cls, shape=shape, dtype=dtype, requires_grad=requires_grad, device=dev)
        MXFP8TensorStorage.__init__(self, rowwise_data=rowwise_data, rowwise_scale_inv=rowwise_scale_inv,
                                    columnwise_data=columnwise_data, columnwise_scale_inv=columnwise_scale_inv,
                                    fp8_dtype=fp8_dtype, quantizer=quantizer, shape=shape, dtype=dtype)
        return self

    def __init__(self, *a, **k):
        pass

    def dequantize(self, *, dtype=None):
        return QuantizedTensor.dequantize(self, dtype=dtype)

    def _new_like(self, requires_grad=None, clone=False, dtype=None):
        c = (lambda t: t.clone() if (clone and t is not None) else t)
        return MXFP8Tensor(shape=self._shape, dtype=dtype or self._dtype, rowwise_data=c(self._rowwise_data),
                           rowwise_scale_inv=c(self._rowwise_scale_inv), columnwise_data=c(self._columnwise_data),
                           columnwise_scale_inv=c(self._columnwise_scale_inv), fp8_dtype=self._fp8_dtype,
                           quantizer=self._quantizer,
                           requires_grad=self.requires_grad if requires_grad is None else requires_grad)

    def __reduce_ex__(self, protocol):
        return (_make_mxfp8_tensor_in_reduce_ex,
                (self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv,
                 self._fp8_dtype, self._dtype, self._shape, None, True))

    # ---- structural ops that keep the MXFP8 payload when FSDP2 shards a parameter along its rows (chunk, padded
    # buffer, copy into a slice).  Only whole 128-row scale tiles can be cut: other requests take the generic
    # (dequantizing) path, and the parameter is then sharded in high precision.  Pieces carry the row-wise copy only.
    def _row_piece(self, r0: int, r1: int) -> "MXFP8Tensor":
        R, C = self._rows_cols()
        per_tile = self._rowwise_scale_inv.numel() // ((R + 127) // 128)
        data = self._rowwise_data.reshape(R, C)[r0:r1]
        sc = self._rowwise_scale_inv.reshape(-1)[(r0 // 128) * per_tile:((r1 + 127) // 128) * per_tile]
        return MXFP8Tensor(shape=(r1 - r0, C), dtype=self._dtype, rowwise_data=data, rowwise_scale_inv=sc,
                           columnwise_data=None, columnwise_scale_inv=None, fp8_dtype=self._fp8_dtype,
                           quantizer=self._quantizer)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        aten = torch.ops.aten
        t = args[0] if args else None
        if isinstance(t, MXFP8Tensor) and t._rowwise_data is not None and len(t._shape) == 2:
            R, C = t._rows_cols()
            if func == aten.split.Tensor and (args[2] if len(args) > 2 else kwargs.get("dim", 0)) == 0 \
                    and isinstance(args[1], int) and args[1] % 128 == 0 and R % 128 == 0:
                return tuple(t._row_piece(r, min(r + args[1], R)) for r in range(0, R, args[1]))
            if func == aten.slice.Tensor:
                dim = args[1] if len(args) > 1 else 0
                start = args[2] if len(args) > 2 and args[2] is not None else 0
                end = min(args[3], R) if len(args) > 3 and args[3] is not None else R
                step = args[4] if len(args) > 4 else 1
                if dim == 0 and step == 1 and start % 128 == 0 and (end % 128 == 0 or end == R) and end > start:
                    return t._row_piece(start, end)
            if func == aten.new_zeros.default and len(args[1]) == 2 and args[1][1] == C and args[1][0] % 128 == 0:
                rows = args[1][0]
                dev = kwargs.get("device") or t._rowwise_data.device
                per_tile = t._rowwise_scale_inv.numel() // ((R + 127) // 128)
                return MXFP8Tensor(shape=(rows, C), dtype=t._dtype,
                                   rowwise_data=torch.zeros(rows, C, dtype=t._rowwise_data.dtype, device=dev),
                                   rowwise_scale_inv=torch.zeros(rows // 128 * per_tile, dtype=torch.uint8, device=dev),
                                   columnwise_data=None, columnwise_scale_inv=None, fp8_dtype=t._fp8_dtype,
                                   quantizer=t._quantizer)
            if func == aten.view.default and tuple(args[1]) in ((-1,), (R * C,)):
                # the flat alias that FSDP2 keeps of a sharded parameter: same buffers, 1-D shape (never computed on)
                return MXFP8Tensor(shape=(R * C,), dtype=t._dtype, rowwise_data=t._rowwise_data,
                                   rowwise_scale_inv=t._rowwise_scale_inv, columnwise_data=None,
                                   columnwise_scale_inv=None, fp8_dtype=t._fp8_dtype, quantizer=t._quantizer)
            if func == aten.as_strided.default and tuple(args[1]) == (R, C) and tuple(args[2]) == (C, 1) \
                    and not (len(args) > 3 and args[3]):
                # FSDP2 restrides the gathered tensor to the parameter's original (contiguous) layout: an alias
                # over the same buffers, so that later all-gathers into them show through the parameter
                return MXFP8Tensor(shape=(R, C), dtype=t._dtype, rowwise_data=t._rowwise_data,
                                   rowwise_scale_inv=t._rowwise_scale_inv, columnwise_data=t._columnwise_data,
                                   columnwise_scale_inv=t._columnwise_scale_inv, fp8_dtype=t._fp8_dtype,
                                   quantizer=t._quantizer)
            if func == aten.copy_.default and isinstance(args[1], MXFP8Tensor) and args[1]._rowwise_data is not None \
                    and tuple(args[1]._shape) == tuple(t._shape) and args[1]._fp8_dtype == t._fp8_dtype:
                src = args[1]
                t._rowwise_data.reshape(R, C).copy_(src._rowwise_data.reshape(R, C))
                t._rowwise_scale_inv.reshape(-1).copy_(src._rowwise_scale_inv.reshape(-1))
                t._columnwise_data = t._columnwise_scale_inv = None
                return t
        return super().__torch_dispatch__(func, types, args, kwargs)

    # ---- FSDP2 extension points (reference: tensor/mxfp8_tensor.py:606-757).  Row shards must be whole
    # 128-row scale tiles; then the row-wise data and its tile-major scales of the shards concatenate
    # byte-wise into the full tensor's, and the column-wise copy is rebuilt after the gather.
    def fsdp_pre_all_gather(self, mesh=None, orig_size=None, contiguous_orig_stride=None, module=None, mp_policy=None):
        assert self._rowwise_data is not None, "FSDP gathers the row-wise copy"
        R, _ = self._rows_cols()
        assert R % 128 == 0, "MXFP8 parameter shards must hold a multiple of 128 rows"
        return ((self._rowwise_data.view(torch.uint8), self._rowwise_scale_inv.reshape(R // 128, -1)),
                (self._fp8_dtype, self._dtype, self._quantizer))

    def fsdp_post_all_gather(self, all_gather_outputs, metadata, param_dtype=None, *, out=None):
        data, scales = all_gather_outputs
        fp8_dtype, dtype, quantizer = metadata
        full = MXFP8Tensor(shape=data.shape, dtype=dtype, rowwise_data=data, rowwise_scale_inv=scales.reshape(-1),
                           columnwise_data=None, columnwise_scale_inv=None, fp8_dtype=fp8_dtype, quantizer=quantizer)
        if out is not None:
            out._rowwise_data, out._rowwise_scale_inv = full._rowwise_data, full._rowwise_scale_inv
            out._columnwise_data = out._columnwise_scale_inv = None
            return None
        return full, all_gather_outputs


def _make_mxfp8_tensor_in_reduce_ex(rowwise_data, rowwise_scale_inv, columnwise_data, columnwise_scale_inv,
                                    fp8_dtype, dtype, shape, quantizer=None, with_gemm_swizzled_scales=True):
    return MXFP8Tensor(shape=shape, dtype=dtype, rowwise_data=rowwise_data, rowwise_scale_inv=rowwise_scale_inv,
                       columnwise_data=columnwise_data, columnwise_scale_inv=columnwise_scale_inv,
                       fp8_dtype=fp8_dtype, quantizer=quantizer)


class MXFP8Quantizer(Quantizer):
    def __init__(self, fp8_dtype: torch.dtype = torch.float8_e4m3fn, *, rowwise=True, columnwise=True,
                 with_2d_quantization: bool = False):
        super().__init__(rowwise=rowwise, columnwise=columnwise)
        self.dtype = fp8_dtype
        # one scale per 32 x 32 block instead of per 1 x 32: both copies then hold the same values (weights)
        self.with_2d_quantization = bool(with_2d_quantization)

    def is_quantizable(self, inp):
        if inp.dim() < 2:
            return False
        C = inp.shape[-1]
        R = inp.numel() // max(C, 1)
        return C % 32 == 0 and R % 32 == 0

    def is_requantization_safe(self) -> bool:
        return True

    def get_scale_shape(self, shape: Iterable[int], columnwise: bool):
        """``(outer, inner)`` extent of the UE8M0 scale buffer of a tensor of ``shape`` (one scale per 32 values,
        padded to whole 128 x 4 tiles; the buffer itself is flat and tile-swizzled).  The column-wise copy is stored
        transposed, so its scales are those of a ``[last dim, rows]`` matrix."""
        shape = tuple(shape)
        C = shape[-1]
        R = 1
        for d in shape[:-1]:
            R *= d
        if columnwise:
            return (Q.round_up(C, 128), Q.round_up(R // 32, 4))
        return (Q.round_up(R, 128), Q.round_up(C // 32, 4))

    def create_tensor_from_data(self, data: torch.Tensor, scale_inv: torch.Tensor,
                                fake_dtype: torch.dtype = torch.float32, fp8_dtype: Optional[torch.dtype] = None,
                                requires_grad: bool = False):
        """Wrap existing row-wise bytes and their (tile-swizzled) scales as a tensor of this quantizer."""
        data = data if data.dtype == torch.uint8 else data.view(torch.uint8)
        outer, inner = self.get_scale_shape(data.shape, False)
        if scale_inv.numel() != outer * inner:
            raise ValueError(f"scale_inv must hold {outer * inner} bytes for data of shape {tuple(data.shape)}")
        return MXFP8Tensor(shape=tuple(data.shape), dtype=fake_dtype, rowwise_data=data,
                           rowwise_scale_inv=scale_inv.reshape(-1), columnwise_data=None, columnwise_scale_inv=None,
                           fp8_dtype=fp8_dtype or self.dtype, quantizer=self, requires_grad=requires_grad)

    def _wrap(self, rd, rs, cd, cs, shape, hp_dtype, requires_grad=False):
        kw = dict(rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd, columnwise_scale_inv=cs,
                  fp8_dtype=self.dtype, quantizer=self, shape=shape, dtype=hp_dtype)
        if self.internal:
            return MXFP8TensorStorage(**kw)
        return MXFP8Tensor(requires_grad=requires_grad, **kw)

    def quantize_impl(self, tensor, dtype=None):
        shape = tuple(tensor.shape)
        x2d = tensor.reshape(-1, shape[-1])
        rd, rs, cd, cs = ops.quantize_mxfp8(x2d, self.dtype, rowwise=self.rowwise_usage,
                                            columnwise=self.columnwise_usage, two_d=self.with_2d_quantization)
        if rd is not None:
            rd = rd.reshape(shape)
        return self._wrap(rd, rs, cd, cs, shape, dtype or tensor.dtype)

    def update_quantized(self, src, dst, *, noop_flag=None):
        shape = tuple(dst._shape)
        rd, rs, cd, cs = ops.quantize_mxfp8(src.reshape(-1, shape[-1]), self.dtype,
                                            rowwise=dst._rowwise_data is not None,
                                            columnwise=dst._columnwise_data is not None,
                                            two_d=self.with_2d_quantization)
        if rd is not None:
            dst._rowwise_data.copy_(rd.reshape(shape))
            dst._rowwise_scale_inv.copy_(rs)
        if cd is not None:
            dst._columnwise_data.copy_(cd)
            dst._columnwise_scale_inv.copy_(cs)
        return dst

    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False,
                   pin_memory: bool = False):
        shape = tuple(shape)
        C = shape[-1]
        R = 1
        for s in shape[:-1]:
            R *= s
        rd = rs = cd = cs = None
        kw = dict(dtype=torch.uint8, device=device, pin_memory=pin_memory)
        if self.rowwise_usage:
            rd = torch.empty(shape, **kw)
            rs = torch.zeros(Q.round_up(R, 128) * Q.round_up(C // 32, 4), **kw)
        if self.columnwise_usage:
            cd = torch.empty(C, R, **kw)
            cs = torch.zeros(Q.round_up(C, 128) * Q.round_up(R // 32, 4), **kw)
        was, self.internal = self.internal, False
        try:
            return self._wrap(rd, rs, cd, cs, shape, dtype, requires_grad)
        finally:
            self.internal = was
