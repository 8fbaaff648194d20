"""Multi-head latent attention, query side: up-projection GEMM + per-head rotary embedding + MXFP8
quantization of the result, behind one call.

The projection runs on this library's tcgen05 GEMM (MXFP8 when the weight is an ``MXFP8Tensor``
primary parameter, 16-bit otherwise); the rotation takes ``cos`` / ``sin`` tables and acts on the
LAST ``cos.shape[-1]`` channels of every head (the ``[no-position | rotary]`` split of latent
attention), pairing channel ``i`` with ``i + d_rot / 2``; the MXFP8 quantizer then writes the rowwise and
columnwise copies that an FP8 attention consumes.
(Reference: ``pytorch/attention/fused_mla_q_uproj.py:34`` over a cuDNN-frontend kernel.)
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..ops import gemm as G
from ..tensor.base import QuantizedTensorStorage
from ..tensor.mxfp8 import MXFP8Quantizer, MXFP8TensorStorage


class FusedMLAQUpProjRopeQuant:
    @classmethod
    def is_supported(cls) -> bool:
        from ..utils.config import get_config

        return get_config().fused_mla_q_uproj

    @staticmethod
    def _rope_last(q: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """q [s, b, nh, d]; cos / sin [s, d_rot] (or broadcastable [s, 1, 1, d_rot])."""
        d_rot = cos.shape[-1]
        if d_rot == 0:
            return q
        cos = cos.reshape(cos.shape[0], 1, 1, d_rot).to(torch.float32)
        sin = sin.reshape(sin.shape[0], 1, 1, d_rot).to(torch.float32)
        keep, rot = q[..., :q.shape[-1] - d_rot], q[..., q.shape[-1] - d_rot:].float()
        x1, x2 = rot[..., :d_rot // 2], rot[..., d_rot // 2:]
        rotated = torch.cat([-x2, x1], dim=-1)
        return torch.cat([keep, (rot * cos + rotated * sin).to(q.dtype)], dim=-1)

    @classmethod
    def run(cls, x: torch.Tensor, w, cos: torch.Tensor, sin: torch.Tensor, s: int, b: int,
            head_dim: Optional[int] = None) -> Tuple[MXFP8TensorStorage, object]:
        """``x`` is ``[s * b, K]`` (or ``[s, b, K]``), ``w`` ``[nh * d, K]``.  Returns the query as an
        MXFP8 tensor of logical shape ``[s, b, nh, d]`` and the activation to keep for the weight
        gradient (MXFP8 columnwise copy on the FP8 path, ``x`` itself otherwise)."""
        x2 = x.reshape(-1, x.shape[-1])
        assert x2.shape[0] == s * b, "x must hold s * b tokens"
        n = w.shape[0]
        d = head_dim if head_dim is not None else cos.shape[-1]
        assert n % d == 0, "the weight's rows must be a whole number of heads"
        if isinstance(w, QuantizedTensorStorage):
            assert isinstance(w, MXFP8TensorStorage), \
                "the fused query up-projection takes an MXFP8 weight; use the unfused path for other recipes"
            xq = MXFP8Quantizer(torch.float8_e4m3fn, rowwise=True, columnwise=True)
            xq.internal = True
            x_q = xq(x2)
            out = G.gemm_nt(G.as_operand(x_q, "rowwise"), G.as_operand(w, "rowwise"), out_dtype=torch.bfloat16)
            x_q.update_usage(rowwise_usage=False, columnwise_usage=True)
            x_saved = x_q
        else:
            out = G.gemm_nt(G.as_operand(x2, "rowwise"), G.as_operand(w.to(x2.dtype), "rowwise"), out_dtype=x2.dtype)
            x_saved = x
        q = cls._rope_last(out.reshape(s, b, n // d, d), cos, sin)
        quantizer = MXFP8Quantizer(torch.float8_e4m3fn, rowwise=True, columnwise=True)
        return quantizer(q.contiguous()), x_saved
