"""Matrix multiplication entry points.

``gemm_nt(a, b)`` computes ``a[M,K] @ b[N,K]^T`` for plain 16-bit tensors or
for quantized operands (per-tensor FP8, MXFP8, NVFP4, block FP8).  On CUDA the
work runs on the tcgen05 kernels in ``csrc/gemm``; on CPU the operands are
dequantized and multiplied in fp32, which is the numerical oracle.

``general_gemm(A, B, layout=...)`` keeps the reference's calling convention
(``pytorch/cpp_extensions/gemm.py:191-224``): ``A`` is the weight, ``B`` the
input, ``TN`` -> ``B @ A^T`` (fprop), ``NN`` -> ``B @ A`` (dgrad), ``NT`` ->
``B^T @ A`` (wgrad).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _ext
from .ref import quant as Q

KIND_F16, KIND_MXFP8, KIND_NVFP4, KIND_FP8 = 0, 1, 2, 3
EPI_NONE, EPI_BIAS, EPI_GELU, EPI_DGELU = 0, 1, 2, 3


@dataclass
class Operand:
    """One GEMM operand with its contraction dim last: ``data [rows, K]``."""

    kind: str  # "hp" | "fp8" | "mxfp8" | "nvfp4" | "blockwise"
    data: torch.Tensor
    scale: Optional[torch.Tensor] = None  # block scales (swizzled) or scale_inv [1]
    fp8_dtype: Optional[torch.dtype] = None
    amax: Optional[torch.Tensor] = None  # NVFP4 global amax
    rows: int = 0
    k: int = 0
    rht: bool = False
    hp_fallback: Optional[torch.Tensor] = None  # dequantized values (set lazily)
    sf_k_tiles: int = 0  # MXFP8 view of a slab of the contraction dim: k-tiles per row tile of the WHOLE tensor


def as_operand(t, usage: str = "rowwise") -> Operand:
    """View a tensor as a GEMM operand.

    ``rowwise``: contract over the last dim of ``t``; operand is ``t2d [R, C]``.
    ``columnwise``: contract over the leading dims; operand is ``t2d^T [C, R]``.
    """
    from ..tensor.float8 import Float8TensorStorage
    from ..tensor.mxfp8 import MXFP8TensorStorage
    from ..tensor.nvfp4 import NVFP4TensorStorage
    from ..tensor.blockwise import Float8BlockwiseQTensorStorage

    from ..tensor.hybrid import HybridQuantizedTensorStorage, IdentityTensorStorage

    row = usage == "rowwise"
    if isinstance(t, HybridQuantizedTensorStorage):  # each direction has its own format
        child = t._rowwise if row else t._columnwise
        assert child is not None, f"hybrid operand lacks the {usage} copy"
        return as_operand(child, usage)
    if isinstance(t, IdentityTensorStorage):
        return as_operand(t._data.reshape(t._shape), usage)
    if isinstance(t, MXFP8TensorStorage):
        R, C = t._rows_cols()
        if row:
            assert t._rowwise_data is not None, "MXFP8 operand lacks the rowwise copy"
            return Operand("mxfp8", t._rowwise_data.reshape(R, C), t._rowwise_scale_inv, t._fp8_dtype, rows=R, k=C)
        if t._columnwise_data is None:
            t.ensure_columnwise()      # a parameter re-gathered by FSDP2 for the backward pass: row-wise bytes only
        assert t._columnwise_data is not None, "MXFP8 operand lacks the columnwise copy"
        return Operand("mxfp8", t._columnwise_data, t._columnwise_scale_inv, t._fp8_dtype, rows=C, k=R)
    if isinstance(t, NVFP4TensorStorage):
        R, C = t._rows_cols()
        if row:
            return Operand("nvfp4", t._rowwise_data.reshape(R, C // 2), t._rowwise_scale_inv, amax=t._amax_rowwise,
                           rows=R, k=C)
        if t._columnwise_data is None:
            t.ensure_columnwise()      # a parameter re-gathered by FSDP2: row-wise bytes only
        return Operand("nvfp4", t._columnwise_data, t._columnwise_scale_inv, amax=t._amax_columnwise, rows=C, k=R,
                       rht=t._columnwise_rht)
    if isinstance(t, Float8TensorStorage):
        R, C = t._rows_cols()
        if row:
            if t._data is None:
                t.update_usage(rowwise_usage=True)
            return Operand("fp8", t._data.reshape(R, C), t._scale_inv, t._fp8_dtype, rows=R, k=C)
        if t._transpose is None:
            t.update_usage(columnwise_usage=True)
        return Operand("fp8", t._transpose, t._scale_inv, t._fp8_dtype, rows=C, k=R)
    if isinstance(t, Float8BlockwiseQTensorStorage):
        # power-of-two block scales exist as UE8M0 tiles too (written by the quantize kernel): the operand then
        # IS an MXFP8 operand; fp32 scales (or tensors quantized on the CPU) multiply in high precision
        R, C = t._rows_cols()
        if not row and t._columnwise_data is None:
            t.ensure_columnwise()      # a parameter re-gathered by FSDP2: row-wise bytes only
        if row and t._rowwise_data is not None and t._rowwise_mx_scale is not None:
            return Operand("mxfp8", t._rowwise_data.reshape(R, C), t._rowwise_mx_scale, t._fp8_dtype, rows=R, k=C)
        if not row and t._columnwise_data is not None and t._columnwise_mx_scale is not None:
            return Operand("mxfp8", t._columnwise_data, t._columnwise_mx_scale, t._fp8_dtype, rows=C, k=R)
        hp = t.dequantize(dtype=torch.bfloat16 if t._dtype == torch.float32 else t._dtype)
        return as_operand(hp, usage)
    t2d = t.reshape(-1, t.shape[-1])
    if row:
        return Operand("hp", t2d, rows=t2d.shape[0], k=t2d.shape[1])
    return Operand("hp", t2d.t(), rows=t2d.shape[1], k=t2d.shape[0])


def contraction_slab(op: Operand, k0: int, k1: int) -> Operand:
    """View of an MXFP8 (or 16-bit) operand restricted to columns ``[k0, k1)`` of its contraction dim, both
    multiples of 128: no copy; block scales are addressed with the whole tensor's tile pitch."""
    assert k0 % 128 == 0 and k1 % 128 == 0 and 0 <= k0 <= k1 <= op.k
    if op.kind == "hp":
        return Operand("hp", op.data[:, k0:k1], rows=op.rows, k=k1 - k0)
    assert op.kind == "mxfp8", "contraction slabs are implemented for MXFP8 and 16-bit operands"
    total = op.sf_k_tiles or (Q.round_up((op.k + 31) // 32, 4) // 4)
    return Operand("mxfp8", op.data[:, k0:k1], op.scale[(k0 // 128) * 512:], op.fp8_dtype, rows=op.rows, k=k1 - k0,
                   sf_k_tiles=total)


def _dequant_operand(op: Operand, dtype=torch.float32) -> torch.Tensor:
    from . import quantize as qz

    if op.kind == "hp":
        return op.data.to(dtype)
    if op.kind == "fp8":
        return qz.dequantize_fp8(op.data, op.scale, op.fp8_dtype, dtype)
    if op.kind == "mxfp8":
        return qz.dequantize_mxfp8(op.data, op.scale, op.fp8_dtype, dtype)
    if op.kind == "nvfp4":
        return qz.dequantize_nvfp4(op.data, op.scale, op.amax, op.rows, op.k, dtype)
    raise ValueError(op.kind)


def _gelu(x):
    return x * (0.5 + 0.5 * torch.tanh(x * (0.79788456 + 0.03567741 * x * x)))


def _dgelu(x):
    t = torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x))
    return 0.5 * x * ((1 - t * t) * (0.79788456 + 0.1070322243 * x * x)) + 0.5 * (1 + t)


def gemm_nt(
    a,
    b,
    *,
    out_dtype: Optional[torch.dtype] = None,
    out: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    epilogue: int = EPI_NONE,
    aux: Optional[torch.Tensor] = None,
    alpha: float = 1.0,
    group_offsets: Optional[torch.Tensor] = None,
    num_groups: int = 0,
    sm_count: int = 0,
) -> torch.Tensor:
    """``D[M,N] = alpha * a[M,K] @ b[N,K]^T (+ bias) (+ D)``; operands are :class:`Operand`."""
    if not isinstance(a, Operand):
        a = as_operand(a, "rowwise")
    if not isinstance(b, Operand):
        b = as_operand(b, "rowwise")
    assert a.k == b.k, f"contraction mismatch {a.k} vs {b.k}"
    M = a.rows
    N = b.rows // num_groups if num_groups else b.rows
    dev = a.data.device
    if out is None:
        if out_dtype is None:
            out_dtype = a.data.dtype if a.kind == "hp" else torch.bfloat16
        out = torch.empty(M, N, dtype=out_dtype, device=dev)
        assert not accumulate, "accumulate needs an output tensor"
    if M == 0 or N == 0:
        return out
    if a.k == 0:
        if not accumulate:
            out.zero_()
        return out
    if _ext.use_cuda(a.data):
        if any(o.kind == "hp" and o.data.dtype in (torch.float32, torch.float64) for o in (a, b)):
            # fp32 operands keep fp32 math (the tcgen05 kernels take 16-bit and narrower inputs and would
            # round them to bf16): library matmul in fp32, same epilogue semantics as the oracle
            return _gemm_ref(a, b, out, bias, accumulate, epilogue, aux, alpha, group_offsets, num_groups)
        return _gemm_cuda(a, b, out, bias, accumulate, epilogue, aux, alpha, group_offsets, num_groups, sm_count)
    return _gemm_ref(a, b, out, bias, accumulate, epilogue, aux, alpha, group_offsets, num_groups)


def _gemm_ref(a, b, out, bias, accumulate, epilogue, aux, alpha, group_offsets, num_groups):
    af = _dequant_operand(a)
    bf = _dequant_operand(b)
    if a.kind == "hp" and a.data.dtype in (torch.bfloat16, torch.float16):
        af, bf = af.float(), bf.float()
    if num_groups:
        offs = group_offsets.tolist()
        N = b.rows // num_groups
        acc = torch.zeros(a.rows, N, dtype=torch.float32, device=af.device)
        for g in range(num_groups):
            acc[offs[g]:offs[g + 1]] = af[offs[g]:offs[g + 1]] @ bf[g * N:(g + 1) * N].t()
    else:
        acc = af @ bf.t()
    acc = acc * alpha
    if bias is not None:
        acc = acc + bias.float()
    if epilogue == EPI_GELU:
        aux.copy_(acc.to(aux.dtype))
        acc = _gelu(acc)
    elif epilogue == EPI_DGELU:
        acc = acc * _dgelu(aux.float())
    if accumulate:
        acc = acc + out.float()
    out.copy_(acc.to(out.dtype))
    return out


_OPERAND_MN_MAJOR = False  # read transposed 16-bit operands in place instead of copying them


def _hp_cuda_operand(op: Operand, dtype) -> Tuple[torch.Tensor, bool]:
    """Return (2-D tensor, mn_major flag) for a 16-bit operand."""
    d = op.data
    if d.dtype != dtype:
        d = d.to(dtype)
    if d.stride(-1) == 1 and d.stride(0) % 8 == 0 and d.data_ptr() % 16 == 0:
        return d, False
    if _OPERAND_MN_MAJOR and d.stride(0) == 1 and d.stride(1) % 8 == 0 and d.data_ptr() % 16 == 0:
        return d.t(), True  # stored [K, rows]
    return d.contiguous(), False


def _gemm_cuda(a, b, out, bias, accumulate, epilogue, aux, alpha, group_offsets, num_groups, sm_count):
    C_ = _ext.get()
    kinds = {a.kind, b.kind}
    alpha_dev = None
    if kinds == {"mxfp8"} and a.k % 32 == 0:
        kind = KIND_MXFP8
        ad, bd = a.data, b.data
        sfa, sfb = a.scale, b.scale
        a_mn = b_mn = False
    elif kinds == {"fp8"} and a.k % 16 == 0 and a.data.is_contiguous() and b.data.is_contiguous():
        kind = KIND_FP8
        ad, bd = a.data.view(torch.uint8), b.data.view(torch.uint8)
        sfa = sfb = None
        a_mn = b_mn = False
        # per-tensor decode scales folded into the epilogue
        alpha_dev = (a.scale.float().reshape(-1)[:1] * b.scale.float().reshape(-1)[:1]).contiguous()
    elif kinds == {"nvfp4"} and a.k % 256 == 0:
        kind = KIND_NVFP4
        ad, bd = a.data, b.data
        sfa, sfb = a.scale, b.scale
        a_mn = b_mn = False
        # fold both tensor-level decode scales into the epilogue
        alpha_dev = (a.amax.float() * b.amax.float()) * (1.0 / (6.0 * 6.0 * 448.0 * 448.0))
    else:
        kind = KIND_F16
        cdt = torch.bfloat16
        for o in (a, b):
            if o.kind == "hp" and o.data.dtype == torch.float16:
                cdt = torch.float16
        ah = a.data if a.kind == "hp" else _dequant_operand(a, cdt)
        bh = b.data if b.kind == "hp" else _dequant_operand(b, cdt)
        ad, a_mn = _hp_cuda_operand(Operand("hp", ah), cdt)
        bd, b_mn = _hp_cuda_operand(Operand("hp", bh), cdt)
        sfa = sfb = None
        K = a.k
        if K % 8 != 0:
            # TMA needs 16-byte row pitch: pad the contraction dim with zeros
            pad = 8 - K % 8
            ad = torch.nn.functional.pad(ad if not a_mn else ad.t(), (0, pad)).contiguous()
            bd = torch.nn.functional.pad(bd if not b_mn else bd.t(), (0, pad)).contiguous()
            a_mn = b_mn = False
    d = out
    direct = d.dim() == 2 and d.stride(1) == 1 and d.dtype in (torch.float32, torch.bfloat16, torch.float16) \
        and (d.stride(0) * d.element_size()) % 16 == 0 and d.data_ptr() % 16 == 0
    if not direct:
        d = torch.empty(out.shape, dtype=torch.float32 if out.dtype not in (torch.bfloat16, torch.float16) else out.dtype,
                        device=out.device)
        if accumulate:
            d.copy_(out)
    if bias is not None and epilogue == EPI_NONE:
        epilogue = EPI_BIAS
    sfk = max(a.sf_k_tiles, b.sf_k_tiles) if kind == KIND_MXFP8 else 0
    if sfk:
        assert a.sf_k_tiles == b.sf_k_tiles, "slab views of the contraction dim must come from equally long tensors"
    C_.gemm(kind, ad, bd, d, sfa, sfb, bias, aux, epilogue, accumulate,
            a.fp8_dtype == torch.float8_e5m2, b.fp8_dtype == torch.float8_e5m2, a_mn, b_mn, float(alpha), alpha_dev,
            group_offsets, num_groups, sm_count, 0, sfk)
    if d is not out:
        out.copy_(d)
    return out


def set_mn_major_operands(flag: bool) -> None:
    """Let 16-bit GEMMs read transposed operands in place (MN-major tcgen05 descriptors)."""
    global _OPERAND_MN_MAJOR
    _OPERAND_MN_MAJOR = bool(flag)


# ----------------------------------------------------------------------------- reference-compatible wrapper
def general_gemm(
    A,
    B,
    workspace=None,
    out_dtype: Optional[torch.dtype] = None,
    quantization_params=None,
    gelu: bool = False,
    gelu_in: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    layout: str = "TN",
    out: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    use_split_accumulator: bool = False,
    grad: bool = False,
    alpha: float = 1.0,
    **_unused,
):
    """Reference-compatible GEMM front end.  Returns (out, bias_grad, gelu_input, extra)."""
    assert layout in ("TN", "NN", "NT"), f"unsupported layout {layout}"
    lead = None
    if layout == "TN":  # out = B @ A^T
        a_op, b_op = as_operand(B, "rowwise"), as_operand(A, "rowwise")
        lead = tuple(B.shape[:-1]) if hasattr(B, "shape") else None
    elif layout == "NN":  # out = B @ A
        a_op, b_op = as_operand(B, "rowwise"), as_operand(A, "columnwise")
        lead = tuple(B.shape[:-1]) if hasattr(B, "shape") else None
    else:  # NT: out = B^T @ A
        a_op, b_op = as_operand(B, "columnwise"), as_operand(A, "columnwise")
    bias_grad = None
    gelu_input = None
    epi, aux = EPI_NONE, None
    if grad and bias is not None:
        # bgrad: column sums of the grad-output operand
        from ..tensor.base import QuantizedTensorStorage as _QS

        src = B.dequantize() if isinstance(B, _QS) else B
        bias_grad = src.reshape(-1, src.shape[-1]).float().sum(0).to(bias.dtype)
        bias = None
    M, N = a_op.rows, b_op.rows
    od = out_dtype or (out.dtype if out is not None else None)
    o2d = out.reshape(M, N) if out is not None else None
    if gelu and not grad:
        aux = torch.empty(M, N, dtype=od or torch.bfloat16, device=a_op.data.device)
        epi, gelu_input = EPI_GELU, aux
    elif gelu and grad:
        epi, aux = EPI_DGELU, gelu_in.reshape(M, N)
    res = gemm_nt(a_op, b_op, out_dtype=od, out=o2d, bias=bias, accumulate=accumulate, epilogue=epi, aux=aux,
                  alpha=alpha)
    if quantization_params is not None:
        res = quantization_params(res)
    elif out is not None:
        res = out
    elif lead is not None and layout != "NT":
        res = res.reshape(*lead, N)
    return res, bias_grad, gelu_input, None
