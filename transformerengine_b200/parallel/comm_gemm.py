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


# Measured on B200 / NVSwitch: one copy CTA (a ring of 32 KB pieces through shared memory) moves about
# 32 GB/s; all of them together saturate near 700 GB/s of the 770 GB/s a peer copy reaches.
_COPY_CTA_BPS, _LINK_BPS, _SMS = 32e9, 700e9, 148


def auto_copy_ctas(gated_bytes: float, side_bytes: float, other_link_bytes: float, flops: float, mxfp8: bool,
                   world: int) -> int:
    """Number of SMs given to copying instead of to the GEMM, from a small time model of the fused kernel.

    ``gated_bytes``: the gathered GEMM operand (peer rows; the GEMM visits the shards in order, so shard i
    must have landed after i / world of the GEMM).  ``side_bytes``: the side gather, which the copy CTAs
    take up once the gated gather is through and which the GEMM CTAs help to finish after their last tile.
    ``other_link_bytes``: inbound NVLink traffic of the GEMM itself (reduce-scatter partials).
    ``TEB200_COPY_CTAS`` overrides the choice."""
    from ..utils.config import get_config

    forced = int(getattr(get_config(), "copy_ctas", 0) or 0)
    if forced > 0:
        return forced
    gemm_rate = 2.4e15 if mxfp8 else 1.3e15
    everyone = min(_SMS * _COPY_CTA_BPS, _LINK_BPS)
    floor = (gated_bytes + other_link_bytes + side_bytes * (world - 1) / world) / _LINK_BPS
    best, best_t = 4, float("inf")
    for c in range(4, 41, 2):
        rate = min(c * _COPY_CTA_BPS, _LINK_BPS)
        t_gemm = max(flops / (gemm_rate * (_SMS - c) / _SMS), (gated_bytes + other_link_bytes) / _LINK_BPS)
        if gated_bytes:
            t_gemm = max(t_gemm, gated_bytes * world / ((world - 1) * rate))
        carried = max(0.0, t_gemm - gated_bytes / rate) * rate
        t = max(t_gemm + max(0.0, side_bytes - carried) / everyone, floor)
        if t < best_t * 0.995:
            best, best_t = c, t
    return best


class SideSpec:
    """Shape of an operand that the copy CTAs of a fused kernel gather next to the GEMM (the
    weight-gradient operand of the layer: what the reference calls bulk overlap,
    ``common/comm_gemm_overlap/comm_gemm_overlap.cpp:444-498``).

    Every rank contributes ``rows x row_bytes`` bytes.  ``interleave=True`` places piece ``s`` at byte
    column ``s * row_bytes`` of a ``[rows, world * row_bytes]`` result (the transposed, column-wise copy
    of a row-sharded MXFP8 tensor, whose ``row_tiles`` scale chunks of ``sf_chunk`` bytes are merged the
    same way); ``interleave=False`` stacks the pieces along the rows (a row-sharded 16-bit tensor)."""

    def __init__(self, rows: int, row_bytes: int, interleave: bool, row_tiles: int = 0, sf_chunk: int = 0):
        assert row_bytes % 16 == 0 and 0 < row_bytes <= 32768, "side gather rows must be 16..32768 bytes, multiple of 16"
        assert sf_chunk % 16 == 0 and sf_chunk <= 32768
        self.rows, self.row_bytes, self.interleave = rows, row_bytes, interleave
        self.row_tiles, self.sf_chunk = row_tiles, sf_chunk

    def key(self):
        return (self.rows, self.row_bytes, self.interleave, self.row_tiles, self.sf_chunk)

    @property
    def data_bytes(self) -> int:
        return self.rows * self.row_bytes

    @property
    def sf_bytes(self) -> int:
        return self.row_tiles * self.sf_chunk

    @staticmethod
    def for_mxfp8_columnwise(C: int, rows_local: int) -> "SideSpec":
        """Column-wise copy ``[C, rows_local]`` (+ swizzled scale tiles) of a row-sharded MXFP8 tensor."""
        assert rows_local % 128 == 0
        return SideSpec(C, rows_local, True, round_up(C, 128) // 128, rows_local // 128 * 512)

    @staticmethod
    def for_rows(rows_local: int, row_bytes: int) -> "SideSpec":
        return SideSpec(rows_local, row_bytes, False)


class _SideStage:
    """Symmetric staging of the side operand (two slots) plus the launch arguments describing it."""

    def __init__(self, buf: SymmetricBuffer, spec: SideSpec, world: int):
        self.spec, self.world = spec, world
        self.stage, self.ptrs = [], []
        for _ in range(2):
            t, p = buf.carve(spec.data_bytes + spec.sf_bytes)
            self.stage.append(t)
            self.ptrs.append(p)

    @staticmethod
    def nbytes(spec: Optional[SideSpec]) -> int:
        return 0 if spec is None else 2 * (spec.data_bytes + spec.sf_bytes + 256)

    def launch_args(self, slot: int, data: torch.Tensor, sf: Optional[torch.Tensor]):
        """Stage this rank's piece and allocate the gathered result.  Returns (kwargs, data_out, sf_out)."""
        sp, w = self.spec, self.world
        st = self.stage[slot]
        flat = data.reshape(-1).view(torch.uint8)
        assert flat.numel() == sp.data_bytes, "side operand does not match the context's shape"
        st[:sp.data_bytes].copy_(flat)
        sf_out = None
        if sp.sf_bytes:
            st[sp.data_bytes:sp.data_bytes + sp.sf_bytes].copy_(sf.reshape(-1).view(torch.uint8)[:sp.sf_bytes])
            sf_out = torch.empty(sp.sf_bytes * w, dtype=torch.uint8, device=st.device)
        if sp.interleave:
            out = torch.empty(sp.rows, w * sp.row_bytes, dtype=torch.uint8, device=st.device)
            pitch, piece_off = w * sp.row_bytes, sp.row_bytes
        else:
            out = torch.empty(w * sp.rows, sp.row_bytes, dtype=torch.uint8, device=st.device)
            pitch, piece_off = sp.row_bytes, sp.rows * sp.row_bytes
        kw = dict(side_src_ptrs=self.ptrs[slot], side_dst=out, side_dst_sf=sf_out,
                  side_geom=[sp.rows, sp.row_bytes, pitch, piece_off, sp.row_tiles, sp.sf_chunk])
        return kw, out, sf_out


class AllGatherGemm:
    """Context of one all-gather -> GEMM site (fixed gathered shape ``[T, K]``)."""

    def __init__(self, group, T: int, K: int, *, mxfp8: bool, dtype=torch.bfloat16,
                 copy_ctas: Optional[int] = None, side: Optional[SideSpec] = None):
        self.group, self.T, self.K, self.mx = group, T, K, mxfp8
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert T % (128 * self.world) == 0, "gathered rows must be a multiple of 128 * tp"
        self.elem = 1 if mxfp8 else torch.empty(0, dtype=dtype).element_size()
        self.dtype = torch.uint8 if mxfp8 else dtype
        self.copy_ctas = copy_ctas   # None: chosen per output width from the bytes to move and the FLOPs
        self._auto: Dict[int, int] = {}
        self.calls = 0
        a_bytes = T * K * self.elem
        sf_bytes = (T // 128) * round_up(K // 32, 4) // 4 * 512 if mxfp8 else 0
        self.sf_bytes = sf_bytes
        nflags = 64 + T // 128
        self.buf = SymmetricBuffer(2 * (a_bytes + sf_bytes + 4 * nflags + 1024) + 4096 + _SideStage.nbytes(side), group)
        self.a, self.a_ptrs, self.sf, self.sf_ptrs = [], [], [], []
        self.ready_ptrs, self.chunk_ptr = [], []
        # Double buffered: a peer may still read call n while call n+1 is staged.  Every slot is a channel
        # of its own (flags included) whose call number is kept on the device by the kernel, so the same
        # launch arguments stay valid when a captured graph replays them.
        for _ in range(2):
            t, p = self.buf.carve(a_bytes)
            self.a.append(t.view(self.dtype).reshape(T, K))
            self.a_ptrs.append(p)
            if mxfp8:
                t, p = self.buf.carve(sf_bytes)
                self.sf.append(t)
                self.sf_ptrs.append(p)
            _, p = self.buf.carve(4 * 64)
            self.ready_ptrs.append(p)
            _, p = self.buf.carve(4 * (T // 128))
            self.chunk_ptr.append(p[self.rank])
        self.epoch_dev = [torch.zeros(4, dtype=torch.int32, device=self.a[0].device) for _ in range(2)]
        self.side = _SideStage(self.buf, side, self.world) if side is not None else None

    def __call__(self, x_local, w, *, bias=None, out_dtype=torch.bfloat16, side=None,
                 timeline: Optional[torch.Tensor] = None):
        """``x_local``: this rank's rows (plain 16-bit tensor or MXFP8 with a rowwise copy);
        ``w``: the local weight ``[N, K]`` of the same kind.  Returns ``[T, N]``; with ``side=(data, scales)``
        (this rank's piece of the side operand) returns ``(out, gathered_data, gathered_scales)``."""
        a_op = x_local if isinstance(x_local, Operand) else as_operand(x_local, "rowwise")
        b_op = w if isinstance(w, Operand) else as_operand(w, "rowwise")
        rows = self.T // self.world
        assert a_op.rows == rows and a_op.k == self.K
        self.calls += 1
        slot = self.calls & 1
        lo = self.rank * rows
        self.a[slot][lo:lo + rows].copy_(a_op.data.view(self.dtype) if self.mx else a_op.data)
        sfa = None
        if self.mx:
            per = self.sf_bytes // self.world
            self.sf[slot][self.rank * per:(self.rank + 1) * per].copy_(a_op.scale[:per])
            sfa = self.sf[slot]
        N = b_op.rows
        out = torch.empty(self.T, N, dtype=out_dtype, device=self.a[slot].device)
        kw, sd, ssf = ({}, None, None) if side is None else self.side.launch_args(slot, side[0], side[1])
        cc = self.copy_ctas
        if cc is None:
            cc = self._auto.get(N)
            if cc is None:
                w = self.world
                gathered = (self.T * self.K * self.elem + self.sf_bytes) * (w - 1) / w
                side_all = 0 if side is None else (self.side.spec.data_bytes + self.side.spec.sf_bytes) * w
                cc = self._auto[N] = auto_copy_ctas(gathered, side_all, 0.0, 2.0 * self.T * self.K * N, self.mx, w)
        _ext.get().comm_gemm(1, self.rank, self.world, self.epoch_dev[slot], cc, self.a[slot], sfa,
                             b_op.data, b_op.scale if self.mx else None, out, bias,
                             a_op.fp8_dtype == torch.float8_e5m2, b_op.fp8_dtype == torch.float8_e5m2,
                             self.a_ptrs[slot], self.sf_ptrs[slot] if self.mx else [], self.ready_ptrs[slot],
                             self.chunk_ptr[slot], [], [], timeline, N, _status(out.device), **kw)
        return out if side is None else (out, sd, ssf)

    def gathered(self) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """The gathered operand of the last call (valid once that call's kernel has run)."""
        slot = self.calls & 1
        return self.a[slot], (self.sf[slot] if self.mx else None)


class GemmReduceScatter:
    """Context of one GEMM -> reduce-scatter site (fixed output shape ``[T, N]`` before scattering)."""

    def __init__(self, group, T: int, N: int, *, dtype=torch.bfloat16, side: Optional[SideSpec] = None,
                 copy_ctas: Optional[int] = None):
        self.group, self.T, self.N, self.dtype = group, T, N, dtype
        self.copy_ctas = copy_ctas   # None: chosen per contraction length (only used with a side gather)
        self._auto: Dict[int, int] = {}
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert T % (128 * self.world) == 0 and N % 8 == 0
        stage_bytes = T * round_up(N, 256) * 2  # one 64 KB record per 128 x 256 output tile
        mbl = T // 128 // self.world
        self.buf = SymmetricBuffer(2 * stage_bytes + 4 * self.world * mbl * 2 + 8192 + _SideStage.nbytes(side), group)
        self.stage_ptrs = []
        for _ in range(2):
            _, p = self.buf.carve(stage_bytes)
            self.stage_ptrs.append(p)
        # one counter array per staging buffer: each call adds 2 * ceil(N/256) per (source, block); the
        # number of calls made on a buffer is kept on the device by the kernel
        self.flag_ptrs = []
        for _ in range(2):
            _, p = self.buf.carve(4 * self.world * mbl)
            self.flag_ptrs.append(p)
        self.calls = 0
        self.epoch_dev = [torch.zeros(4, dtype=torch.int32, device=self.buf.tensor.device) for _ in range(2)]
        self.side, self.ready_ptrs = None, [[], []]
        if side is not None:
            self.side = _SideStage(self.buf, side, self.world)
            self.ready_ptrs = [self.buf.carve(4 * 64)[1] for _ in range(2)]

    def __call__(self, x, w, *, bias=None, timeline: Optional[torch.Tensor] = None, side=None):
        """``x`` [T, K/tp], ``w`` [N, K/tp] (16-bit or MXFP8 rowwise).  Returns this rank's ``[T/tp, N]``; with
        ``side=(data, scales)`` returns ``(out, gathered_data, gathered_scales)``."""
        a_op = x if isinstance(x, Operand) else as_operand(x, "rowwise")
        b_op = w if isinstance(w, Operand) else as_operand(w, "rowwise")
        assert a_op.rows == self.T and b_op.rows == self.N
        self.calls += 1
        slot = self.calls & 1
        mx = a_op.kind == "mxfp8"
        out = torch.empty(self.T // self.world, self.N, dtype=self.dtype, device=a_op.data.device)
        kw, sd, ssf = ({}, None, None) if side is None else self.side.launch_args(slot, side[0], side[1])
        cc = 0
        if side is not None:
            cc = self.copy_ctas
            if cc is None:
                cc = self._auto.get(a_op.k)
                if cc is None:
                    w = self.world
                    side_all = (self.side.spec.data_bytes + self.side.spec.sf_bytes) * w
                    partial_in = self.T * self.N * 2 * (w - 1) / w      # what the peers push into this rank
                    cc = self._auto[a_op.k] = auto_copy_ctas(0.0, side_all, partial_in,
                                                             2.0 * self.T * self.N * a_op.k, mx, w)
        _ext.get().comm_gemm(2, self.rank, self.world, self.epoch_dev[slot], cc,
                             a_op.data, a_op.scale if mx else None,
                             b_op.data, b_op.scale if mx else None, timeline, bias,
                             a_op.fp8_dtype == torch.float8_e5m2, b_op.fp8_dtype == torch.float8_e5m2,
                             [], [], self.ready_ptrs[slot], 0, self.stage_ptrs[slot], self.flag_ptrs[slot], out, self.N,
                             _status(out.device), **kw)
        return out if side is None else (out, sd, ssf)


class GemmAllReduce:
    """Context of one GEMM -> all-reduce site (row-parallel layer without sequence parallelism): every rank ends
    with the full ``[T, N]`` sum.  The reduce-scatter kernel with a tail that writes this rank's reduced rows into
    the result buffer of every rank and returns when all ranks' rows have arrived.  The result is a view of a
    double-buffered symmetric buffer: it stays valid until the second next call on this context.
    (Reference: the GEMM + all-reduce of ``common/include/transformer_engine/comm_gemm.h:138``.)"""

    def __init__(self, group, T: int, N: int, *, dtype=torch.bfloat16):
        self.group, self.T, self.N, self.dtype = group, T, N, dtype
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert T % (128 * self.world) == 0 and N % 8 == 0
        stage_bytes = T * round_up(N, 256) * 2
        out_bytes = T * N * 2
        mbl = T // 128 // self.world
        self.buf = SymmetricBuffer(2 * (stage_bytes + out_bytes + 4 * self.world * mbl + 4 * 64) + 8192, group)
        self.stage_ptrs, self.flag_ptrs, self.out, self.out_ptrs, self.ar_ptrs = [], [], [], [], []
        for _ in range(2):
            _, p = self.buf.carve(stage_bytes)
            self.stage_ptrs.append(p)
            _, p = self.buf.carve(4 * self.world * mbl)
            self.flag_ptrs.append(p)
            t, p = self.buf.carve(out_bytes)
            self.out.append(t.view(dtype).reshape(T, N))
            self.out_ptrs.append(p)
            _, p = self.buf.carve(4 * 64)
            self.ar_ptrs.append(p)
        self.calls = 0
        self.epoch_dev = [torch.zeros(4, dtype=torch.int32, device=self.buf.tensor.device) for _ in range(2)]

    def __call__(self, x, w, *, bias=None):
        """``x`` [T, K/tp], ``w`` [N, K/tp] (16-bit or MXFP8 rowwise).  Returns the summed ``[T, N]``."""
        a_op = x if isinstance(x, Operand) else as_operand(x, "rowwise")
        b_op = w if isinstance(w, Operand) else as_operand(w, "rowwise")
        assert a_op.rows == self.T and b_op.rows == self.N
        self.calls += 1
        slot = self.calls & 1
        mx = a_op.kind == "mxfp8"
        out = self.out[slot]
        _ext.get().comm_gemm(3, self.rank, self.world, self.epoch_dev[slot], 0,
                             a_op.data, a_op.scale if mx else None, b_op.data, b_op.scale if mx else None, None, bias,
                             a_op.fp8_dtype == torch.float8_e5m2, b_op.fp8_dtype == torch.float8_e5m2,
                             [], [], [], 0, self.stage_ptrs[slot], self.flag_ptrs[slot], out, self.N,
                             _status(out.device), out_all_ptrs=self.out_ptrs[slot], ar_flag_ptrs=self.ar_ptrs[slot])
        return out


# --------------------------------------------------------------------------- registry (initialize_ub equivalent)
_CONTEXTS: Dict[tuple, object] = {}
_ENABLED = {"group": None}


def initialize_ub(shape=None, tp_size: Optional[int] = None, use_fp8: bool = False, dtype=torch.bfloat16,
                  ub_cfgs=None, bootstrap_backend=None, tp_group=None, quantization_modes=None,
                  with_cublasmp: bool = False, **_unused) -> None:
    """Turn on fused collective GEMMs for tensor-parallel modules of ``tp_group``.

    Contexts (symmetric buffers + flags) are created lazily per call site and shape.
    """
    if with_cublasmp:
        raise NotImplementedError("with_cublasmp: the collective GEMMs of this library are its own kernels over "
                                  "symmetric memory; there is no cuBLASMp path")
    _ENABLED["group"] = tp_group if tp_group is not None else dist.group.WORLD


def destroy_ub() -> None:
    _CONTEXTS.clear()
    _ENABLED["group"] = None


def is_ub_initialized() -> bool:
    """Whether ``initialize_ub`` has switched the fused collective GEMMs on."""
    return _ENABLED["group"] is not None


def enabled_for(group) -> bool:
    return _ENABLED["group"] is not None and group is not None and _ENABLED["group"] == group


def get_all_gather_gemm(name: str, group, T: int, K: int, mxfp8: bool, dtype,
                        side: Optional[SideSpec] = None) -> AllGatherGemm:
    key = ("ag", name, T, K, mxfp8, dtype, side.key() if side is not None else None)
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        ctx = _CONTEXTS[key] = AllGatherGemm(group, T, K, mxfp8=mxfp8, dtype=dtype, side=side)
    return ctx


def get_gemm_all_reduce(name: str, group, T: int, N: int, dtype) -> GemmAllReduce:
    key = ("ar", name, T, N, dtype)
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        ctx = _CONTEXTS[key] = GemmAllReduce(group, T, N, dtype=dtype)
    return ctx


def get_gemm_reduce_scatter(name: str, group, T: int, N: int, dtype,
                            side: Optional[SideSpec] = None) -> GemmReduceScatter:
    key = ("rs", name, T, N, dtype, side.key() if side is not None else None)
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        ctx = _CONTEXTS[key] = GemmReduceScatter(group, T, N, dtype=dtype, side=side)
    return ctx
