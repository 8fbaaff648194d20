"""NVFP4 tensors: E2M1 data, E4M3 scale per 16 values, fp32 amax per tensor.

Payload (reference layout, ``pytorch/tensor/nvfp4_tensor.py:272-327``):
  ``_rowwise_data``   uint8 ``[R, C/2]``;  ``_rowwise_scale_inv`` E4M3 bytes, swizzled,
  padded ``[ru(R,128) * ru(C/16,4)]``;  ``_amax_rowwise`` fp32 ``[1]``
  ``_columnwise_data`` uint8 ``[C, R/2]`` (transposed); ``_columnwise_scale_inv``
  padded ``[ru(C,128) * ru(R/16,4)]``; ``_amax_columnwise`` fp32 ``[1]``.
With the random Hadamard transform the columnwise copy holds ``RHT(x^T)``:
blocks of 16 tokens are rotated by a fixed signed 16x16 Hadamard matrix, which
cancels in the wgrad GEMM because both operands carry the same rotation.
"""
from __future__ import annotations

from typing import Tuple, Iterable, Optional

import torch

from .. import ops
from ..ops.ref import quant as Q
from .base import QuantizedTensor, QuantizedTensorStorage, Quantizer, pin_payload


class NVFP4TensorStorage(QuantizedTensorStorage):
    def __init__(self, *, rowwise_data, rowwise_scale_inv, columnwise_data, columnwise_scale_inv,
                 amax_rowwise, amax_columnwise, fp4_dtype=None, quantizer=None, shape=None,
                 dtype=torch.float32, columnwise_rht=False):
        self._rowwise_data = rowwise_data
        self._rowwise_scale_inv = rowwise_scale_inv
        self._columnwise_data = columnwise_data
        self._columnwise_scale_inv = columnwise_scale_inv
        self._amax_rowwise = amax_rowwise
        self._amax_columnwise = amax_columnwise
        self._fp4_dtype = fp4_dtype
        self._quantizer = quantizer
        self._dtype = dtype
        self._columnwise_rht = columnwise_rht
        if shape is None:
            if rowwise_data is not None:
                shape = tuple(rowwise_data.shape[:-1]) + (rowwise_data.shape[-1] * 2,)
            else:
                shape = (columnwise_data.shape[1] * 2, columnwise_data.shape[0])
        self._shape = tuple(shape)

    def get_data_tensors(self):
        return self._rowwise_data, self._columnwise_data

    def get_usages(self):
        return {"rowwise": self._rowwise_data is not None, "columnwise": self._columnwise_data is not None}

    def update_usage(self, rowwise_usage=None, columnwise_usage=None):
        if rowwise_usage and self._rowwise_data is None:
            raise RuntimeError("NVFP4 tensor has no rowwise copy")
        if columnwise_usage and self._columnwise_data is None:
            raise RuntimeError("NVFP4 tensor has no columnwise copy")
        if rowwise_usage is False:
            self._rowwise_data = self._rowwise_scale_inv = self._amax_rowwise = None
        if columnwise_usage is False:
            self._columnwise_data = self._columnwise_scale_inv = self._amax_columnwise = None

    def ensure_columnwise(self) -> None:
        """Build the column-wise copy from the row-wise one when it is missing (a parameter gathered by FSDP2 carries
        the row-wise bytes only).  Weights use 16 x 16 blocks without the Hadamard transform, for which both copies
        hold the same values, so re-quantizing the dequantized row-wise copy reproduces what a direct quantization
        gives; with 1-D blocks it is a second rounding along the other direction."""
        if self._columnwise_data is not None or self._rowwise_data is None or len(self._shape) != 2:
            return
        q = self._quantizer
        R, C = self._rows_cols()
        if q is None or R % 16 or C % 16:
            return
        hp = ops.dequantize_nvfp4(self._rowwise_data.reshape(R, C // 2), self._rowwise_scale_inv, self._amax_rowwise,
                                  R, C, torch.bfloat16)
        two_d = bool(getattr(q, "with_2d_quantization", False))
        _, _, _, cd, cs, ac = ops.quantize_nvfp4(hp, rowwise=False, columnwise=True, with_rht=False, with_2d=two_d)
        self._columnwise_data, self._columnwise_scale_inv, self._amax_columnwise = cd, cs, ac
        self._columnwise_rht = False

    def _dequantize_impl(self, dtype=None):
        dtype = dtype or self._dtype
        R, C = self._rows_cols()
        if self._rowwise_data is not None:
            out = ops.dequantize_nvfp4(self._rowwise_data.reshape(R, C // 2), self._rowwise_scale_inv,
                                       self._amax_rowwise, R, C, dtype)
            return out.reshape(self._shape)
        out_t = ops.dequantize_nvfp4(self._columnwise_data, self._columnwise_scale_inv,
                                     self._amax_columnwise, C, R, torch.float32)
        if self._columnwise_rht:
            # the Hadamard matrix with signs is orthogonal: undo with its transpose
            h = Q.hadamard_matrix_16(out_t.device)
            out_t = (out_t.reshape(C, R // 16, 16) @ h.t()).reshape(C, R)
        return out_t.t().contiguous().reshape(self._shape).to(dtype)

    def dequantize(self, *, dtype=None):
        return self._dequantize_impl(dtype)

    def prepare_for_saving(self):
        ts = [self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv,
              self._amax_rowwise, self._amax_columnwise]
        self._rowwise_data = self._rowwise_scale_inv = self._columnwise_data = None
        self._columnwise_scale_inv = self._amax_rowwise = self._amax_columnwise = None
        return ts, self

    def restore_from_saved(self, tensors):
        (self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv,
         self._amax_rowwise, self._amax_columnwise) = tensors[:6]
        return tensors[6:]


class NVFP4Tensor(NVFP4TensorStorage, QuantizedTensor):
    def __new__(cls, *, shape, dtype, rowwise_data, rowwise_scale_inv, columnwise_data, columnwise_scale_inv,
                amax_rowwise, amax_columnwise, fp4_dtype=None, quantizer=None, requires_grad=False,
                device=None, columnwise_rht=False):
        dev = device if device is not None else (rowwise_data if rowwise_data is not None else columnwise_data).device
        self = QuantizedTensor.__new__(cls, shape=shape, dtype=dtype, requires_grad=requires_grad, device=dev)
        NVFP4TensorStorage.__init__(self, rowwise_data=rowwise_data, rowwise_scale_inv=rowwise_scale_inv,
                                    columnwise_data=columnwise_data, columnwise_scale_inv=columnwise_scale_inv,
                                    amax_rowwise=amax_rowwise, amax_columnwise=amax_columnwise,
                                    fp4_dtype=fp4_dtype, quantizer=quantizer, shape=shape, dtype=dtype,
                                    columnwise_rht=columnwise_rht)
        return self

    def __init__(self, *a, **k):
        pass

    def dequantize(self, *, dtype=None):
        return QuantizedTensor.dequantize(self, dtype=dtype)

    def _new_like(self, requires_grad=None, clone=False, dtype=None):
        c = (lambda t: t.clone() if (clone and t is not None) else t)
        return NVFP4Tensor(shape=self._shape, dtype=dtype or self._dtype, rowwise_data=c(self._rowwise_data),
                           rowwise_scale_inv=c(self._rowwise_scale_inv), columnwise_data=c(self._columnwise_data),
                           columnwise_scale_inv=c(self._columnwise_scale_inv), amax_rowwise=c(self._amax_rowwise),
                           amax_columnwise=c(self._amax_columnwise), fp4_dtype=self._fp4_dtype,
                           quantizer=self._quantizer, columnwise_rht=self._columnwise_rht,
                           requires_grad=self.requires_grad if requires_grad is None else requires_grad)

    def __reduce_ex__(self, protocol):
        return (_make_nvfp4_tensor_in_reduce_ex,
                (self._rowwise_data, self._rowwise_scale_inv, self._columnwise_data, self._columnwise_scale_inv,
                 self._amax_rowwise, self._amax_columnwise, self._fp4_dtype, self._dtype, self._shape,
                 self._columnwise_rht))


    # ---- FSDP2 (``fully_shard``): the parameter is cut along its rows into whole 128-row scale tiles; a piece
    # carries the row-wise bytes, its slice of the tile-major E4M3 scales and the tensor amax (shared: one decode
    # scale per tensor).  Same structural ops as the MXFP8 tensor; anything else takes the generic (dequantizing)
    # path and the parameter is then sharded in high precision.
    def _alias(self, shape, data, scales) -> "NVFP4Tensor":
        return NVFP4Tensor(shape=shape, dtype=self._dtype, rowwise_data=data, rowwise_scale_inv=scales,
                           columnwise_data=None, columnwise_scale_inv=None, amax_rowwise=self._amax_rowwise,
                           amax_columnwise=None, fp4_dtype=self._fp4_dtype, quantizer=self._quantizer)

    def _row_piece(self, r0: int, r1: int) -> "NVFP4Tensor":
        R, C = self._rows_cols()
        per_tile = self._rowwise_scale_inv.numel() // ((R + 127) // 128)
        data = self._rowwise_data.reshape(R, C // 2)[r0:r1]
        sc = self._rowwise_scale_inv.reshape(-1)[(r0 // 128) * per_tile:((r1 + 127) // 128) * per_tile]
        return self._alias((r1 - r0, C), data, sc)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        aten = torch.ops.aten
        t = args[0] if args else None
        if isinstance(t, NVFP4Tensor) and t._rowwise_data is not None and len(t._shape) == 2 \
                and t._amax_rowwise is not None:
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
                out = t._alias((rows, C), torch.zeros(rows, C // 2, dtype=torch.uint8, device=dev),
                               torch.zeros(rows // 128 * per_tile, dtype=torch.uint8, device=dev))
                out._amax_rowwise = t._amax_rowwise.clone().to(dev)
                return out
            if func == aten.view.default and tuple(args[1]) in ((-1,), (R * C,)):
                # the flat alias that FSDP2 keeps of a sharded parameter: same buffers, never computed on
                return t._alias((R * C,), t._rowwise_data, t._rowwise_scale_inv)
            if func == aten.as_strided.default and tuple(args[1]) == (R, C) and tuple(args[2]) == (C, 1) \
                    and not (len(args) > 3 and args[3]):
                out = t._alias((R, C), t._rowwise_data, t._rowwise_scale_inv)
                out._columnwise_data, out._columnwise_scale_inv = t._columnwise_data, t._columnwise_scale_inv
                out._amax_columnwise, out._columnwise_rht = t._amax_columnwise, t._columnwise_rht
                return out
            if func == aten.copy_.default and isinstance(args[1], NVFP4Tensor) and args[1]._rowwise_data is not None \
                    and tuple(args[1]._shape) == tuple(t._shape):
                src = args[1]
                t._rowwise_data.reshape(R, C // 2).copy_(src._rowwise_data.reshape(R, C // 2))
                t._rowwise_scale_inv.reshape(-1).copy_(src._rowwise_scale_inv.reshape(-1))
                t._amax_rowwise.copy_(src._amax_rowwise)
                t._columnwise_data = t._columnwise_scale_inv = t._amax_columnwise = None
                return t
        return super().__torch_dispatch__(func, types, args, kwargs)

    def fsdp_pre_all_gather(self, mesh=None, orig_size=None, contiguous_orig_stride=None, module=None, mp_policy=None):
        assert self._rowwise_data is not None, "FSDP gathers the row-wise copy"
        R, C = self._rows_cols()
        assert R % 128 == 0, "NVFP4 parameter shards must hold a multiple of 128 rows"
        q = self._quantizer
        if mesh is not None and q is not None and not q.with_amax_reduction:
            # one decode scale per tensor: re-quantizations of a shard (the optimizer's write-back) take the amax
            # over all shards from now on
            q.with_amax_reduction, q.amax_reduction_group = True, mesh.get_group(mesh.ndim - 1)
        return ((self._rowwise_data.reshape(R, C // 2), self._rowwise_scale_inv.reshape(R // 128, -1)),
                (self._amax_rowwise, self._fp4_dtype, self._dtype, self._quantizer))

    def fsdp_post_all_gather(self, all_gather_outputs, metadata, param_dtype=None, *, out=None):
        data, scales = all_gather_outputs
        amax, fp4_dtype, dtype, quantizer = metadata
        if out is not None:
            out._rowwise_data, out._rowwise_scale_inv, out._amax_rowwise = data, scales.reshape(-1), amax
            out._columnwise_data = out._columnwise_scale_inv = out._amax_columnwise = None
            return None
        full = NVFP4Tensor(shape=(data.shape[0], data.shape[1] * 2), dtype=dtype, rowwise_data=data,
                           rowwise_scale_inv=scales.reshape(-1), columnwise_data=None, columnwise_scale_inv=None,
                           amax_rowwise=amax, amax_columnwise=None, fp4_dtype=fp4_dtype, quantizer=quantizer)
        return full, all_gather_outputs


def _make_nvfp4_tensor_in_reduce_ex(rd, rs, cd, cs, ar, ac, fp4_dtype, dtype, shape, columnwise_rht=False):
    return NVFP4Tensor(shape=shape, dtype=dtype, rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd,
                       columnwise_scale_inv=cs, amax_rowwise=ar, amax_columnwise=ac, fp4_dtype=fp4_dtype,
                       columnwise_rht=columnwise_rht)


class NVFP4Quantizer(Quantizer):
    """NVFP4 builder.

    ``with_rht`` rotates the columnwise (transposed) copy; ``with_2d_quantization``
    uses 16x16 blocks (weights) so that the rowwise and columnwise copies
    dequantize to the same values; ``stochastic_rounding`` for gradients.
    """

    def __init__(self, fp4_dtype=None, *, rowwise=True, columnwise=True, with_amax_reduction=False,
                 amax_reduction_group=None, with_rht=False, with_post_rht_amax=True,
                 with_2d_quantization=False, stochastic_rounding=False, with_random_sign_mask=True,
                 row_scaled_nvfp4: bool = False, nvfp4_use_4over6: bool = False, nvfp4_e4m3_max: int = 448,
                 nvfp4_4over6_err_mode: str = "MAE"):
        super().__init__(rowwise=rowwise, columnwise=columnwise)
        if row_scaled_nvfp4:
            raise NotImplementedError("row_scaled_nvfp4 (one tensor scale per row) is not implemented: the GEMM "
                                      "epilogues apply one scale per operand")
        nvfp4_4over6_err_mode = str(nvfp4_4over6_err_mode).upper()
        if nvfp4_use_4over6:
            if nvfp4_4over6_err_mode not in ("MAE", "MSE"):
                raise ValueError(f"nvfp4_4over6_err_mode must be 'MAE' or 'MSE', got {nvfp4_4over6_err_mode!r}")
            if with_rht or stochastic_rounding:
                raise NotImplementedError("4-over-6 NVFP4 scaling does not combine with the Hadamard transform or "
                                          "stochastic rounding")
            if nvfp4_e4m3_max not in (256, 448):
                raise ValueError("nvfp4_e4m3_max must be 256 or 448")
        self.row_scaled_nvfp4 = False
        self.nvfp4_use_4over6 = bool(nvfp4_use_4over6)
        self.nvfp4_e4m3_max = int(nvfp4_e4m3_max) if nvfp4_use_4over6 else 448
        self.nvfp4_4over6_err_mode = nvfp4_4over6_err_mode
        if with_rht and not with_random_sign_mask:
            raise NotImplementedError("the Hadamard transform always uses the fixed random sign vector "
                                      "(with_random_sign_mask=False is not implemented)")
        self.dtype = fp4_dtype
        self.with_amax_reduction = with_amax_reduction
        self.amax_reduction_group = amax_reduction_group
        self.with_rht = with_rht
        self.with_post_rht_amax = with_post_rht_amax
        self.with_2d_quantization = with_2d_quantization
        self.stochastic_rounding = stochastic_rounding
        self.generator: Optional[torch.Generator] = None

    def is_quantizable(self, inp):
        if inp.dim() < 2:
            return False
        C = inp.shape[-1]
        R = inp.numel() // max(C, 1)
        return C % 16 == 0 and R % 16 == 0

    def is_requantization_safe(self) -> bool:
        return not self.stochastic_rounding

    def get_scale_shape(self, shape: Iterable[int], columnwise: bool):
        """``(outer, inner)`` extent of the E4M3 block-scale buffer of a tensor of ``shape`` (one scale per 16
        values, padded to whole 128 x 4 tiles; the buffer itself is flat and tile-swizzled).  The column-wise copy
        is stored transposed."""
        shape = tuple(shape)
        C = shape[-1]
        R = 1
        for d in shape[:-1]:
            R *= d
        if columnwise:
            R, C = C, R
        return (Q.round_up(R, 128), Q.round_up(C // 16, 4))

    @staticmethod
    def convert_shape_for_fp4(shape: Iterable[int]) -> Tuple[int, ...]:
        """Shape of the packed byte buffer of a tensor of ``shape``: two E2M1 values per byte along the last dim."""
        shape = tuple(shape)
        if shape[-1] % 2:
            raise ValueError(f"the last dimension must be even to pack FP4 pairs, got {shape}")
        return shape[:-1] + (shape[-1] // 2,)

    def _reduce(self, amax):
        if self.with_amax_reduction and self.amax_reduction_group is not None:
            torch.distributed.all_reduce(amax, op=torch.distributed.ReduceOp.MAX, group=self.amax_reduction_group)
        return amax

    def _wrap(self, parts, shape, hp_dtype, requires_grad=False):
        rd, rs, ar, cd, cs, ac = parts
        kw = dict(rowwise_data=rd, rowwise_scale_inv=rs, columnwise_data=cd, columnwise_scale_inv=cs,
                  amax_rowwise=ar, amax_columnwise=ac, fp4_dtype=self.dtype, quantizer=self, shape=shape,
                  dtype=hp_dtype, columnwise_rht=self.with_rht)
        if self.internal:
            return NVFP4TensorStorage(**kw)
        return NVFP4Tensor(requires_grad=requires_grad, **kw)

    def _quantize_parts(self, x2d, rowwise, columnwise):
        return ops.quantize_nvfp4(x2d, rowwise=rowwise, columnwise=columnwise, with_rht=self.with_rht,
                                  with_2d=self.with_2d_quantization, stochastic_rounding=self.stochastic_rounding,
                                  amax_reduce=self._reduce, generator=self.generator,
                                  four_over_six=self.nvfp4_4over6_err_mode if self.nvfp4_use_4over6 else None,
                                  e4m3_max=float(self.nvfp4_e4m3_max))

    def quantize_impl(self, tensor, dtype=None):
        shape = tuple(tensor.shape)
        parts = self._quantize_parts(tensor.reshape(-1, shape[-1]), self.rowwise_usage, self.columnwise_usage)
        rd = parts[0]
        if rd is not None:
            parts = (rd.reshape(shape[:-1] + (shape[-1] // 2,)),) + tuple(parts[1:])
        return self._wrap(parts, shape, dtype or tensor.dtype)

    def update_quantized(self, src, dst, *, noop_flag=None):
        shape = tuple(dst._shape)
        rd, rs, ar, cd, cs, ac = self._quantize_parts(src.reshape(-1, shape[-1]), dst._rowwise_data is not None,
                                                     dst._columnwise_data is not None)
        if rd is not None:
            dst._rowwise_data.copy_(rd.reshape(dst._rowwise_data.shape))
            dst._rowwise_scale_inv.copy_(rs)
            dst._amax_rowwise.copy_(ar)
        if cd is not None:
            dst._columnwise_data.copy_(cd)
            dst._columnwise_scale_inv.copy_(cs)
            dst._amax_columnwise.copy_(ac)
        return dst

    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False,
                   pin_memory: bool = False):
        shape = tuple(shape)
        C = shape[-1]
        R = 1
        for s in shape[:-1]:
            R *= s
        rd = rs = ar = cd = cs = ac = None
        if self.rowwise_usage:
            rd = torch.empty(shape[:-1] + (C // 2,), dtype=torch.uint8, device=device)
            rs = torch.zeros(Q.round_up(R, 128) * Q.round_up(C // 16, 4), dtype=torch.uint8, device=device)
            ar = torch.zeros(1, dtype=torch.float32, device=device)
        if self.columnwise_usage:
            cd = torch.empty(C, R // 2, dtype=torch.uint8, device=device)
            cs = torch.zeros(Q.round_up(C, 128) * Q.round_up(R // 16, 4), dtype=torch.uint8, device=device)
            ac = torch.zeros(1, dtype=torch.float32, device=device)
        was, self.internal = self.internal, False
        try:
            out = self._wrap((rd, rs, ar, cd, cs, ac), shape, dtype, requires_grad)
        finally:
            self.internal = was
        return pin_payload(out) if pin_memory else out
