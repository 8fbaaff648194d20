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

    def ensure_columnwise(self) -> None:
        """Build the column-wise copy from the row-wise one when it is missing (a parameter gathered by FSDP2 carries
        the row-wise bytes only).  With 128 x 128 blocks (weights) both copies hold the same values, so this equals
        a direct quantization; with 1 x 128 blocks it is a second rounding along the other direction."""
        if self._columnwise_data is not None or self._rowwise_data is None or len(self._shape) != 2 \
                or self._quantizer is None:
            return
        q = self._quantizer.copy()
        q.set_usage(rowwise=False, columnwise=True)
        q.internal = True
        tmp = q.quantize_impl(self._dequantize_impl(torch.bfloat16 if self._dtype == torch.float32 else self._dtype))
        self._columnwise_data, self._columnwise_scale_inv = tmp._columnwise_data, tmp._columnwise_scale_inv
        self._columnwise_mx_scale = tmp._columnwise_mx_scale

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


    # ---- FSDP2 (``fully_shard``): the parameter is cut along its rows into whole 128-row blocks; a piece carries the
    # row-wise bytes, the matching rows of the fp32 block scales and (when the quantize kernel wrote them) of the
    # tile-major UE8M0 scales.  Other cuts take the generic (dequantizing) path.
    def _alias(self, shape, data, scales, mx) -> "Float8BlockwiseQTensor":
        out = Float8BlockwiseQTensor(shape=shape, dtype=self._dtype, rowwise_data=data, rowwise_scale_inv=scales,
                                     columnwise_data=None, columnwise_scale_inv=None, fp8_dtype=self._fp8_dtype,
                                     is_2D_scaled=self._is_2D_scaled, quantizer=self._quantizer)
        out._rowwise_mx_scale = mx
        return out

    def _row_piece(self, r0: int, r1: int) -> "Float8BlockwiseQTensor":
        R, C = self._rows_cols()
        br = 128 if self._is_2D_scaled else 1
        mx = self._rowwise_mx_scale
        if mx is not None:
            per_tile = mx.numel() // ((R + 127) // 128)
            mx = mx.reshape(-1)[(r0 // 128) * per_tile:((r1 + 127) // 128) * per_tile]
        return self._alias((r1 - r0, C), self._rowwise_data.reshape(R, C)[r0:r1],
                           self._rowwise_scale_inv[r0 // br:-(-r1 // br)], mx)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        aten = torch.ops.aten
        t = args[0] if args else None
        if isinstance(t, Float8BlockwiseQTensor) and t._rowwise_data is not None and len(t._shape) == 2:
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
                br = 128 if t._is_2D_scaled else 1
                mx = t._rowwise_mx_scale
                if mx is not None:
                    mx = torch.zeros(rows // 128 * (mx.numel() // ((R + 127) // 128)), dtype=torch.uint8, device=dev)
                return t._alias((rows, C), torch.zeros(rows, C, dtype=t._rowwise_data.dtype, device=dev),
                                torch.ones(rows // br, t._rowwise_scale_inv.shape[1], dtype=torch.float32, device=dev),
                                mx)
            if func == aten.view.default and tuple(args[1]) in ((-1,), (R * C,)):
                return t._alias((R * C,), t._rowwise_data, t._rowwise_scale_inv, t._rowwise_mx_scale)
            if func == aten.as_strided.default and tuple(args[1]) == (R, C) and tuple(args[2]) == (C, 1) \
                    and not (len(args) > 3 and args[3]):
                out = t._alias((R, C), t._rowwise_data, t._rowwise_scale_inv, t._rowwise_mx_scale)
                out._columnwise_data, out._columnwise_scale_inv = t._columnwise_data, t._columnwise_scale_inv
                out._columnwise_mx_scale = t._columnwise_mx_scale
                return out
            if func == aten.copy_.default and isinstance(args[1], Float8BlockwiseQTensor) \
                    and args[1]._rowwise_data is not None and tuple(args[1]._shape) == tuple(t._shape) \
                    and args[1]._is_2D_scaled == t._is_2D_scaled:
                src = args[1]
                t._rowwise_data.reshape(R, C).copy_(src._rowwise_data.reshape(R, C))
                t._rowwise_scale_inv.copy_(src._rowwise_scale_inv)
                if t._rowwise_mx_scale is not None and src._rowwise_mx_scale is not None:
                    t._rowwise_mx_scale.reshape(-1).copy_(src._rowwise_mx_scale.reshape(-1))
                else:
                    t._rowwise_mx_scale = None
                t._columnwise_data = t._columnwise_scale_inv = t._columnwise_mx_scale = None
                return t
        return super().__torch_dispatch__(func, types, args, kwargs)

    def fsdp_pre_all_gather(self, mesh=None, orig_size=None, contiguous_orig_stride=None, module=None, mp_policy=None):
        assert self._rowwise_data is not None, "FSDP gathers the row-wise copy"
        R, C = self._rows_cols()
        assert R % 128 == 0, "block-scaled parameter shards must hold a multiple of 128 rows"
        parts = [self._rowwise_data.reshape(R, C).view(torch.uint8),
                 self._rowwise_scale_inv.contiguous().view(torch.uint8)]          # fp32 scales travel as bytes
        if self._rowwise_mx_scale is not None:
            parts.append(self._rowwise_mx_scale.reshape(R // 128, -1))
        return tuple(parts), (self._fp8_dtype, self._is_2D_scaled, self._dtype, self._quantizer)

    def fsdp_post_all_gather(self, all_gather_outputs, metadata, param_dtype=None, *, out=None):
        data, scales = all_gather_outputs[0], all_gather_outputs[1].view(torch.float32)
        mx = all_gather_outputs[2].reshape(-1) if len(all_gather_outputs) > 2 else None
        fp8_dtype, is_2d, dtype, quantizer = metadata
        if out is not None:
            out._rowwise_data, out._rowwise_scale_inv, out._rowwise_mx_scale = data, scales, mx
            out._columnwise_data = out._columnwise_scale_inv = out._columnwise_mx_scale = None
            return None
        full = Float8BlockwiseQTensor(shape=tuple(data.shape), dtype=dtype, rowwise_data=data, rowwise_scale_inv=scales,
                                      columnwise_data=None, columnwise_scale_inv=None, fp8_dtype=fp8_dtype,
                                      is_2D_scaled=is_2d, quantizer=quantizer)
        full._rowwise_mx_scale = mx
        return full, all_gather_outputs


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
