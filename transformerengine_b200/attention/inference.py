"""KV cache for incremental decoding: ``InferenceParams`` with a contiguous (non-paged) and a
paged cache manager (reference: ``pytorch/attention/inference.py:57, 405, 596``).

Usage, per generation step::

    params = InferenceParams(max_batch_size=8, max_sequence_length=4096, num_heads_kv=8,
                             head_dim_k=128, dtype=torch.bfloat16, is_paged=True, page_size=64,
                             total_num_pages=512)
    params.pre_step(OrderedDict((seq_id, new_tokens) ...))   # which sequences advance, by how much
    y = transformer_layer(x, inference_params=params, ...)      # every layer calls params.step(...)

``step`` appends the new K/V tokens of the step to the layer's cache and hands attention the
packed ("thd") queries together with every sequence's full cached K/V and the cumulative
lengths, so that the causal mask is aligned bottom-right per sequence.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch

from . import thd as _thd


def _step_metadata(lens_old: List[int], lens_new: List[int], tables: List[List[int]], device):
    """Device-side description of one decoding step, shared by all layers: page table
    ``[sequences, width]`` (-1 where unused) and the cumulative new / resulting lengths."""
    width = max((len(t) for t in tables), default=1) or 1
    pt = [list(t) + [-1] * (width - len(t)) for t in tables]
    cu_new, cu_kv = [0], [0]
    for o, n in zip(lens_old, lens_new):
        cu_new.append(cu_new[-1] + n)
        cu_kv.append(cu_kv[-1] + o + n)
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=device)  # noqa: E731
    return mk(pt).reshape(len(tables), width), mk(cu_new), mk(cu_kv), cu_kv[-1]


class KVCacheManager:
    """Interface of a cache manager (custom managers may subclass it)."""

    def reset(self) -> None:
        """Forget every sequence (the cache memory stays allocated)."""
        raise NotImplementedError

    def allocate_memory(self, layer_number: int) -> None:
        raise NotImplementedError

    def pre_step(self, step_dict: "OrderedDict[int, int]") -> None:
        raise NotImplementedError

    def step(self, layer_number: int, new_k: torch.Tensor, new_v: torch.Tensor, cu_new: List[int]):
        """Append packed new tokens ``[t_new, h, d]``; return packed full K, V and their lengths."""
        raise NotImplementedError


class NonPagedKVCacheManager(KVCacheManager):
    """One ``[max_batch, max_seq, h, d]`` slab per layer; a sequence owns one batch slot."""

    def __init__(self, max_batch_size, max_sequence_length, num_heads_kv, head_dim_k, dtype, head_dim_v=None,
                 device=None):
        self.max_batch_size, self.max_seq = max_batch_size, max_sequence_length
        self.h, self.dk, self.dv = num_heads_kv, head_dim_k, head_dim_v or head_dim_k
        self.dtype, self.device = dtype, device
        self.cache: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.slots: "OrderedDict[int, int]" = OrderedDict()   # seq id -> batch slot
        self.lengths: Dict[int, int] = {}                       # seq id -> tokens cached BEFORE this step
        self.step_dict: "OrderedDict[int, int]" = OrderedDict()
        self.free_slots = list(range(max_batch_size - 1, -1, -1))
        self._meta = None  # device metadata of the current step (built by the first layer)

    def allocate_memory(self, layer_number):
        dev = self.device or ("cuda" if torch.cuda.is_available() else "cpu")
        k = torch.zeros(self.max_batch_size, self.max_seq, self.h, self.dk, dtype=self.dtype, device=dev)
        v = torch.zeros(self.max_batch_size, self.max_seq, self.h, self.dv, dtype=self.dtype, device=dev)
        self.cache[layer_number] = (k, v)

    def pre_step(self, step_dict):
        # sequences that are not part of this step have finished: release their slots
        for sid in [s for s in self.slots if s not in step_dict]:
            self.free_slots.append(self.slots.pop(sid))
            self.lengths.pop(sid, None)
        for sid in step_dict:
            if sid not in self.slots:
                assert self.free_slots, "KV cache is full: more live sequences than max_batch_size"
                self.slots[sid] = self.free_slots.pop()
                self.lengths[sid] = 0
        self.step_dict = OrderedDict(step_dict)
        self._meta = None

    def post_step(self):
        for sid, n in self.step_dict.items():
            self.lengths[sid] += n

    def reset(self) -> None:
        self.slots.clear()
        self.lengths.clear()
        self.step_dict = OrderedDict()
        self.free_slots = list(range(self.max_batch_size - 1, -1, -1))
        self._meta = None

    def step(self, layer_number, new_k, new_v, cu_new):
        if layer_number not in self.cache:
            self.allocate_memory(layer_number)
        kc, vc = self.cache[layer_number]
        olds = [self.lengths[sid] for sid in self.step_dict]
        news = list(self.step_dict.values())
        assert all(o + n <= self.max_seq for o, n in zip(olds, news)), "sequence exceeds max_sequence_length"
        if self._meta is None or self._meta[0].device != kc.device:
            # the whole slab is one "page" per slot: page size = max_seq, page table = slot
            self._meta = _step_metadata(olds, news, [[self.slots[sid]] for sid in self.step_dict], kc.device)
        pt, cu_n, cu_kv, total = self._meta
        k, v = _thd.kv_cache_step(new_k[:cu_new[-1]], new_v[:cu_new[-1]], kc, vc, pt, cu_n, cu_kv, total)
        return k, v, [o + n for o, n in zip(olds, news)]


class PagedKVCacheManager(KVCacheManager):
    """Pages of ``page_size`` tokens shared by all sequences, a page table per sequence."""

    def __init__(self, total_num_pages, page_size, num_heads_kv, head_dim_k, dtype, max_batch_size,
                 max_sequence_length, head_dim_v=None, device=None):
        self.total_num_pages, self.page_size = total_num_pages, page_size
        self.h, self.dk, self.dv = num_heads_kv, head_dim_k, head_dim_v or head_dim_k
        self.dtype, self.device = dtype, device
        self.max_batch_size, self.max_seq = max_batch_size, max_sequence_length
        self.cache: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.free_pages = list(range(total_num_pages - 1, -1, -1))
        self.page_table: "OrderedDict[int, List[int]]" = OrderedDict()
        self.lengths: Dict[int, int] = {}
        self.step_dict: "OrderedDict[int, int]" = OrderedDict()
        self._meta = None

    def allocate_memory(self, layer_number):
        dev = self.device or ("cuda" if torch.cuda.is_available() else "cpu")
        k = torch.zeros(self.total_num_pages, self.page_size, self.h, self.dk, dtype=self.dtype, device=dev)
        v = torch.zeros(self.total_num_pages, self.page_size, self.h, self.dv, dtype=self.dtype, device=dev)
        self.cache[layer_number] = (k, v)

    def pre_step(self, step_dict):
        for sid in [s for s in self.page_table if s not in step_dict]:
            self.free_pages.extend(self.page_table.pop(sid))
            self.lengths.pop(sid, None)
        for sid, n in step_dict.items():
            if sid not in self.page_table:
                assert len(self.page_table) < self.max_batch_size, "more live sequences than max_batch_size"
                self.page_table[sid] = []
                self.lengths[sid] = 0
            need = -(-(self.lengths[sid] + n) // self.page_size) - len(self.page_table[sid])
            assert need <= len(self.free_pages), "KV cache is out of pages"
            for _ in range(max(need, 0)):
                self.page_table[sid].append(self.free_pages.pop())
        self.step_dict = OrderedDict(step_dict)
        self._meta = None

    def post_step(self):
        for sid, n in self.step_dict.items():
            self.lengths[sid] += n

    def get_page_table(self, sequences: Optional[List[int]] = None, device=None) -> torch.Tensor:
        """``[num_sequences, max_pages_per_seq]`` int32 table of the live sequences (or of ``sequences``, in that
        order), -1 where unused."""
        tables = [self.page_table[s] for s in sequences] if sequences is not None else list(self.page_table.values())
        width = max((len(p) for p in tables), default=0)
        t = torch.full((len(tables), width), -1, dtype=torch.int32, device=device)
        for i, pages in enumerate(tables):
            t[i, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        return t

    # ---- bookkeeping queries and manual page management (reference: attention/inference.py, PagedKVCacheManager)
    def reset(self) -> None:
        self.free_pages = list(range(self.total_num_pages - 1, -1, -1))
        self.page_table = OrderedDict()
        self.lengths = {}
        self.step_dict = OrderedDict()
        self._meta = None

    def get_sequence_count(self) -> int:
        return len(self.page_table)

    def get_sequence_lengths(self) -> List[int]:
        """Cached tokens of every live sequence (before the step in flight)."""
        return [self.lengths[s] for s in self.page_table]

    def has_free_page(self) -> bool:
        return len(self.free_pages) > 0

    def get_page_count(self, seq: int) -> int:
        return len(self.page_table.get(seq, ()))

    def get_page_list(self, seq: int) -> List[int]:
        return list(self.page_table.get(seq, ()))

    def allocate_page(self, seq: int) -> None:
        if not self.free_pages:
            raise RuntimeError("KV cache is full!")
        self.page_table.setdefault(seq, []).append(self.free_pages.pop())
        self.lengths.setdefault(seq, 0)

    def allocate_sequence(self, seq: int, context_len: int) -> None:
        """Reserve the pages ``context_len`` tokens of a new sequence need."""
        for _ in range(-(-context_len // self.page_size)):
            self.allocate_page(seq)

    def deallocate_sequence(self, seq: int) -> None:
        self.free_pages.extend(self.page_table.pop(seq, ()))
        self.lengths.pop(seq, None)

    def print_cache(self) -> None:
        import logging

        log = logging.getLogger("PagedKVCacheManager")
        used = sum(len(p) for p in self.page_table.values())
        log.debug("total pages: %s (used %s, free %s); sequences: %s", self.total_num_pages, used,
                  len(self.free_pages), len(self.page_table))
        for i, (seq, pages) in enumerate(self.page_table.items()):
            log.debug("  batch index %s: seq_id %s, tokens %s, pages %s", i, seq, self.lengths.get(seq, 0), pages)

    def step(self, layer_number, new_k, new_v, cu_new):
        if layer_number not in self.cache:
            self.allocate_memory(layer_number)
        kc, vc = self.cache[layer_number]
        olds = [self.lengths[sid] for sid in self.step_dict]
        news = list(self.step_dict.values())
        if self._meta is None or self._meta[0].device != kc.device:
            self._meta = _step_metadata(olds, news, [self.page_table[sid] for sid in self.step_dict], kc.device)
        pt, cu_n, cu_kv, total = self._meta
        k, v = _thd.kv_cache_step(new_k[:cu_new[-1]], new_v[:cu_new[-1]], kc, vc, pt, cu_n, cu_kv, total)
        return k, v, [o + n for o, n in zip(olds, news)]


class InferenceParams:
    """State of incremental decoding shared by all layers of a model."""

    def __init__(self, max_batch_size: int, max_sequence_length: int, num_heads_kv: Optional[int] = None,
                 head_dim_k: Optional[int] = None, dtype: Optional[torch.dtype] = None,
                 head_dim_v: Optional[int] = None, is_paged: bool = False, total_num_pages: Optional[int] = None,
                 page_size: Optional[int] = None, max_ctx_len: Optional[int] = None, qkv_format: str = "bshd",
                 custom_cache_manager=None, device=None):
        self.max_batch_size, self.max_sequence_length = max_batch_size, max_sequence_length
        self.num_heads_kv, self.head_dim_k, self.head_dim_v = num_heads_kv, head_dim_k, head_dim_v or head_dim_k
        self.dtype, self.is_paged, self.page_size = dtype, is_paged, page_size
        self.total_num_pages, self.max_ctx_len, self.input_qkv_format = total_num_pages, max_ctx_len, qkv_format
        if custom_cache_manager is not None:
            self.cache_manager = custom_cache_manager
        elif is_paged:
            assert page_size and total_num_pages, "a paged cache needs page_size and total_num_pages"
            self.cache_manager = PagedKVCacheManager(total_num_pages, page_size, num_heads_kv, head_dim_k, dtype,
                                                     max_batch_size, max_sequence_length, head_dim_v, device)
        else:
            self.cache_manager = NonPagedKVCacheManager(max_batch_size, max_sequence_length, num_heads_kv,
                                                        head_dim_k, dtype, head_dim_v, device)
        self.step_dict: "OrderedDict[int, int]" = OrderedDict()
        self.sequences: "OrderedDict[int, int]" = OrderedDict()   # seq id -> length before the current step
        self._layers_seen: set = set()
        self._pending_post = False
        self._orig: Optional[Tuple[str, int, int]] = None

    # ---- step bookkeeping
    def reset(self):
        self.pre_step(OrderedDict())
        self.sequences = OrderedDict()
        if hasattr(self.cache_manager, "reset"):
            try:
                self.cache_manager.reset()
            except NotImplementedError:
                pass

    def allocate_memory(self, layer_number: int):
        self.cache_manager.allocate_memory(layer_number)

    def pre_step(self, step_dict: "OrderedDict[int, int]"):
        if self._pending_post:
            self.cache_manager.post_step()
            self._pending_post = False
        self.cache_manager.pre_step(step_dict)
        self.step_dict = OrderedDict(step_dict)
        self.sequences = OrderedDict((sid, self.cache_manager.lengths[sid]) for sid in step_dict)
        self._layers_seen = set()
        self._pending_post = bool(step_dict)

    def get_seqlens_pre_step(self) -> torch.Tensor:
        return torch.tensor(list(self.sequences.values()), dtype=torch.int32)

    def convert_paged_to_nonpaged(self, layer_number: int):
        """The paged cache of one layer as contiguous ``[sequences, pages_per_seq * page_size, h, d]`` tensors
        (sequences in batch order; positions past a sequence's length hold whatever its last page holds)."""
        assert self.is_paged, "the cache is not paged"
        k, v = self.cache_manager.cache[layer_number]
        table = self.cache_manager.get_page_table(device=k.device).clamp(min=0).long()
        n, w = table.shape
        gather = lambda c: c[table.reshape(-1)].reshape(n, w * c.shape[1], *c.shape[2:]).contiguous()  # noqa: E731
        return gather(k), gather(v)

    def __repr__(self) -> str:
        kind = f"paged (page_size={self.page_size}, total_num_pages={self.total_num_pages})" if self.is_paged \
            else "non-paged"
        return (f"InferenceParams({kind}, max_batch_size={self.max_batch_size}, "
                f"max_sequence_length={self.max_sequence_length}, num_heads_kv={self.num_heads_kv}, "
                f"head_dim_k={self.head_dim_k}, head_dim_v={self.head_dim_v}, dtype={self.dtype}, "
                f"sequences={dict(self.sequences)})")

    def sequence_start_positions(self, batch: int, device) -> torch.Tensor:
        """Position of each sequence's first new token (RoPE offset)."""
        starts = list(self.sequences.values())
        starts += [0] * (batch - len(starts))
        return torch.tensor(starts[:batch], dtype=torch.int32, device=device)

    # ---- per-layer cache update
    def step(self, layer_number, q, k, v, qkv_format, mask_type):
        """Returns (q, k, v, "thd", mask type, cu_seqlens_q, cu_seqlens_kv) for attention."""
        lens_new = list(self.step_dict.values())
        nb = len(lens_new)
        if qkv_format == "thd":
            cu = [0]
            for n in lens_new:
                cu.append(cu[-1] + n)
            qp, kp, vp = q, k[:cu[-1]], v[:cu[-1]]
            self._orig = ("thd", q.shape[0], 0)
        else:
            if qkv_format == "sbhd":
                q, k, v = (t.transpose(0, 1) for t in (q, k, v))
            b, s = q.shape[0], q.shape[1]
            assert nb <= b, "step_dict names more sequences than the batch holds"
            cu = [0]
            for n in lens_new:
                cu.append(cu[-1] + n)
            cu_t = torch.tensor(cu, dtype=torch.int32, device=q.device)
            qp, kp, vp = (_thd.convert_bshd_to_thd(t, cu_t, cu[-1]) for t in (q, k, v))
            self._orig = (qkv_format, b, s)
            self._cu_new = cu_t
        kf, vf, lens_kv = self.cache_manager.step(layer_number, kp, vp, cu)
        cu_kv = [0]
        for n in lens_kv:
            cu_kv.append(cu_kv[-1] + n)
        dev = q.device
        mt = "padding_causal_bottom_right" if "causal" in mask_type else "padding"
        return (qp, kf, vf, "thd", mt, torch.tensor(cu, dtype=torch.int32, device=dev),
                torch.tensor(cu_kv, dtype=torch.int32, device=dev))

    def unpack_output(self, out: torch.Tensor) -> torch.Tensor:
        """Packed attention output ``[t, h*d]`` back to the layout the caller passed in."""
        fmt, b, s = self._orig
        if fmt == "thd":
            return out
        res = _thd.convert_thd_to_bshd(out, self._cu_new, b, s)
        return res.transpose(0, 1) if fmt == "sbhd" else res
