"""GEMMs fused with their tensor-parallel collective over NVLink peer memory.

``AllGatherGemm``:   ``Y[T, N] = all_gather_rows(X_local) @ W^T``  (column-parallel fprop,
row-parallel dgrad).  ``GemmReduceScatter``: ``Y[T/tp, N] = reduce_scatter(X @ W^T)``
(row-parallel fprop, column-parallel dgrad).  One kernel does the math and the transfer
(``csrc/comm/comm_gemm.cu``); buffers live in symmetric memory obtained from
``torch.distributed._symmetric_memory`` (used only to allocate and exchange addresses).
This replaces the reference's ``initialize_ub`` / Userbuffers overlap
(``pytorch/module/base.py:151-514``).

On CPU tensors (gloo) the same classes run the collective and the GEMM one after the
other, which is the oracle for the GPU tests.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops.gemm import Operand, as_operand, gemm_nt
from ..ops.ref.quant import round_up
from . import distributed as D


class SymmetricBuffer:
    """A byte buffer of equal size on every rank of ``group`` whose peer addresses are known."""

    def __init__(self, nbytes: int, group, device=None):
        import torch.distributed._symmetric_memory as symm

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        dev = device or torch.device("cuda", torch.cuda.current_device())
        nbytes = round_up(nbytes, 256)
        self.tensor = symm.empty(nbytes, dtype=torch.uint8, device=dev)
        self.handle = symm.rendezvous(self.tensor, group)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier(group)
        self._off = 0
        self.nbytes = nbytes

    def carve(self, nbytes: int) -> Tuple[torch.Tensor, List[int]]:
        """Next ``nbytes`` of the buffer: (local uint8 view, that region's address on every rank)."""
        off = round_up(self._off, 256)
        assert off + nbytes <= self.nbytes, "symmetric workspace exhausted"
        self._off = off + nbytes
        return self.tensor[off:off + nbytes], [p + off for p in self.ptrs]


def _status(dev) -> torch.Tensor:
    return _ext.get().status(dev.index if dev.index is not None else torch.cuda.current_device())


class AllGatherGemm:
    """Context of one all-gather -> GEMM site (fixed gathered shape ``[T, K]``)."""

    def __init__(self, group, T: int, K: int, *, mxfp8: bool, dtype=torch.bfloat16, copy_ctas: int = 12):
        self.group, self.T, self.K, self.mx = group, T, K, mxfp8
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert T % (128 * self.world) == 0, "gathered rows must be a multiple of 128 * tp"
        self.elem = 1 if mxfp8 else torch.empty(0, dtype=dtype).element_size()
        self.dtype = torch.uint8 if mxfp8 else dtype
        self.copy_ctas = copy_ctas
        self.epoch = 0
        a_bytes = T * K * self.elem
        sf_bytes = (T // 128) * round_up(K // 32, 4) // 4 * 512 if mxfp8 else 0
        self.sf_bytes = sf_bytes
        nflags = 256 + T // 128
        self.buf = SymmetricBuffer(2 * (a_bytes + sf_bytes) + 4 * nflags + 4096, group)
        self.a, self.a_ptrs, self.sf, self.sf_ptrs = [], [], [], []
        for _ in range(2):  # double buffered: a peer may still read call n while call n+1 is staged
            t, p = self.buf.carve(a_bytes)
            self.a.append(t.view(self.dtype).reshape(T, K))
            self.a_ptrs.append(p)
            if mxfp8:
                t, p = self.buf.carve(sf_bytes)
                self.sf.append(t)
                self.sf_ptrs.append(p)
        self.ready, self.ready_ptrs = self.buf.carve(4 * 64)
        self.chunk, chunk_ptrs = self.buf.carve(4 * (T // 128))
        self.chunk_ptr = chunk_ptrs[self.rank]

    def __call__(self, x_local, w, *, bias=None, out_dtype=torch.bfloat16) -> torch.Tensor:
        """``x_local``: this rank's rows (plain 16-bit tensor or MXFP8 with a rowwise copy);
        ``w``: the local weight ``[N, K]`` of the same kind.  Returns ``[T, N]``."""
        a_op = x_local if isinstance(x_local, Operand) else as_operand(x_local, "rowwise")
        b_op = w if isinstance(w, Operand) else as_operand(w, "rowwise")
        rows = self.T // self.world
        assert a_op.rows == rows and a_op.k == self.K
        self.epoch += 1
        slot = self.epoch & 1
        lo = self.rank * rows
        self.a[slot][lo:lo + rows].copy_(a_op.data.view(self.dtype) if self.mx else a_op.data)
        sfa = None
        if self.mx:
            per = self.sf_bytes // self.world
            self.sf[slot][self.rank * per:(self.rank + 1) * per].copy_(a_op.scale[:per])
            sfa = self.sf[slot]
        N = b_op.rows
        out = torch.empty(self.T, N, dtype=out_dtype, device=self.a[slot].device)
        _ext.get().comm_gemm(1, self.rank, self.world, self.epoch, self.copy_ctas, self.a[slot], sfa, b_op.data,
                             b_op.scale if self.mx else None, out, bias,
                             a_op.fp8_dtype == torch.float8_e5m2, b_op.fp8_dtype == torch.float8_e5m2,
                             self.a_ptrs[slot], self.sf_ptrs[slot] if self.mx else [], self.ready_ptrs,
                             self.chunk_ptr, [], [], None, N, _status(out.device))
        return out

    def gathered(self) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """The gathered operand of the last call (valid once that call's kernel has run)."""
        slot = self.epoch & 1
        return self.a[slot], (self.sf[slot] if self.mx else None)


class GemmReduceScatter:
    """Context of one GEMM -> reduce-scatter site (fixed output shape ``[T, N]`` before scattering)."""

    def __init__(self, group, T: int, N: int, *, dtype=torch.bfloat16):
        self.group, self.T, self.N, self.dtype = group, T, N, dtype
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert T % (128 * self.world) == 0 and N % 8 == 0
        self.epoch = 0
        stage_bytes = T * round_up(N, 256) * 2  # one 64 KB record per 128 x 256 output tile
        mbl = T // 128 // self.world
        self.buf = SymmetricBuffer(2 * stage_bytes + 4 * self.world * mbl * 2 + 4096, group)
        self.stage_ptrs = []
        for _ in range(2):
            _, p = self.buf.carve(stage_bytes)
            self.stage_ptrs.append(p)
        # one counter array per staging buffer: each call adds ceil(N/256) per (source, block)
        self.flag_ptrs = []
        for _ in range(2):
            _, p = self.buf.carve(4 * self.world * mbl)
            self.flag_ptrs.append(p)
        self.calls = [0, 0]

    def __call__(self, x, w, *, bias=None, timeline: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` [T, K/tp], ``w`` [N, K/tp] (16-bit or MXFP8 rowwise).  Returns this rank's ``[T/tp, N]``."""
        a_op = x if isinstance(x, Operand) else as_operand(x, "rowwise")
        b_op = w if isinstance(w, Operand) else as_operand(w, "rowwise")
        assert a_op.rows == self.T and b_op.rows == self.N
        self.epoch += 1
        slot = self.epoch & 1
        self.calls[slot] += 1
        mx = a_op.kind == "mxfp8"
        out = torch.empty(self.T // self.world, self.N, dtype=self.dtype, device=a_op.data.device)
        _ext.get().comm_gemm(2, self.rank, self.world, self.calls[slot], 0, a_op.data, a_op.scale if mx else None,
                             b_op.data, b_op.scale if mx else None, timeline, bias,
                             a_op.fp8_dtype == torch.float8_e5m2, b_op.fp8_dtype == torch.float8_e5m2,
                             [], [], [], 0, self.stage_ptrs[slot], self.flag_ptrs[slot], out, self.N,
                             _status(out.device))
        return out


# --------------------------------------------------------------------------- registry (initialize_ub equivalent)
_CONTEXTS: Dict[tuple, object] = {}
_ENABLED = {"group": None}


def initialize_ub(shape=None, tp_size: Optional[int] = None, use_fp8: bool = False, dtype=torch.bfloat16,
                  ub_cfgs=None, bootstrap_backend=None, tp_group=None, quantization_modes=None, **_unused) -> None:
    """Turn on fused collective GEMMs for tensor-parallel modules of ``tp_group``.

    Contexts (symmetric buffers + flags) are created lazily per call site and shape.
    """
    _ENABLED["group"] = tp_group if tp_group is not None else dist.group.WORLD


def destroy_ub() -> None:
    _CONTEXTS.clear()
    _ENABLED["group"] = None


def enabled_for(group) -> bool:
    return _ENABLED["group"] is not None and group is not None and _ENABLED["group"] == group


def get_all_gather_gemm(name: str, group, T: int, K: int, mxfp8: bool, dtype) -> AllGatherGemm:
    key = ("ag", name, T, K, mxfp8, dtype)
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        ctx = _CONTEXTS[key] = AllGatherGemm(group, T, K, mxfp8=mxfp8, dtype=dtype)
    return ctx


def get_gemm_reduce_scatter(name: str, group, T: int, N: int, dtype) -> GemmReduceScatter:
    key = ("rs", name, T, N, dtype)
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        ctx = _CONTEXTS[key] = GemmReduceScatter(group, T, N, dtype=dtype)
    return ctx
