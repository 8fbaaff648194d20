"""Packed-sequence ("thd") helpers: context-parallel partitioning, merging of partial softmax
states, thd <-> bshd conversion and the fused KV-cache step.

On CUDA tensors every function is one kernel of ``csrc/misc/thd.cu``; the PyTorch bodies below are
the CPU path and the oracle of the kernel tests.  Context-parallel convention: every sequence is cut
into ``2 * cp`` equal chunks and rank ``r`` holds chunks ``r`` and ``2 * cp - 1 - r`` -- the "first
half" and "second half" of its local tokens.  LSE tensors are ``[heads, tokens]`` fp32.
(Reference counterparts: ``pytorch/csrc/extensions/attention.cpp:792-1088``.)
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from ..ops import _ext

_MODES = {"none": 0, "copy": 1, "add": 2}


def _cuda(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda for t in ts) and _ext.available() and hasattr(_ext.get(), "kv_cache_step")


def _cu32(cu: torch.Tensor, device) -> torch.Tensor:
    return cu.to(device=device, dtype=torch.int32).contiguous()


def _half_index(cu_seqlens: torch.Tensor, half_idx: int, total: int) -> torch.Tensor:
    """Token indices of the chosen half of every sequence (``total`` = packed length, may exceed cu[-1])."""
    cu = cu_seqlens.tolist()
    idx: List[int] = []
    for a, b in zip(cu[:-1], cu[1:]):
        hl = (b - a) // 2
        idx.extend(range(a + half_idx * hl, a + half_idx * hl + hl))
    pad = total // 2 - len(idx)
    if pad > 0:  # padding tokens after the last sequence: keep the count, pick in-range tokens
        idx.extend(range(cu[-1] + half_idx * pad, cu[-1] + half_idx * pad + pad))
    return torch.tensor(idx, dtype=torch.long)


def thd_get_partitioned_indices(cu_seqlens: torch.Tensor, total_tokens: int, world_size: int, rank: int) -> torch.Tensor:
    """Indices (into the full packed tensor) of the tokens that context-parallel rank ``rank`` holds."""
    assert total_tokens % (2 * world_size) == 0 and 0 <= rank < world_size
    if _cuda(cu_seqlens):
        return _ext.get().thd_get_partitioned_indices(_cu32(cu_seqlens, cu_seqlens.device), total_tokens, world_size, rank)
    cu = cu_seqlens.tolist()
    idx: List[int] = []
    for a, b in zip(cu[:-1], cu[1:]):
        c = (b - a) // (2 * world_size)
        idx.extend(range(a + rank * c, a + rank * c + c))
        idx.extend(range(a + (2 * world_size - 1 - rank) * c, a + (2 * world_size - rank) * c))
    pad = total_tokens // world_size - len(idx)
    if pad > 0:
        idx.extend(range(cu[-1] + rank * pad, cu[-1] + rank * pad + pad))
    return torch.tensor(idx, dtype=torch.int32, device=cu_seqlens.device)


def thd_read_half_tensor(tensor: torch.Tensor, cu_seqlens: torch.Tensor, half_idx: int) -> torch.Tensor:
    """First (0) or second (1) half of every sequence; ``tensor`` is ``[t, h, d]`` or stacked ``[2, t, h, d]``."""
    stacked = tensor.dim() == 4
    if _cuda(tensor):
        return _ext.get().thd_read_half_tensor(tensor, _cu32(cu_seqlens, tensor.device), half_idx, stacked)
    idx = _half_index(cu_seqlens, half_idx, tensor.shape[1 if stacked else 0]).to(tensor.device)
    return tensor.index_select(1 if stacked else 0, idx)


def thd_second_half_lse_correction(lse: torch.Tensor, lse_per_step: torch.Tensor, cu_seqlens: torch.Tensor) -> None:
    """In place: ``lse[:, second halves] = logaddexp(lse[:, second halves], lse_per_step)``."""
    if _cuda(lse, lse_per_step):
        _ext.get().thd_second_half_lse_correction(lse, lse_per_step, _cu32(cu_seqlens, lse.device))
        return
    idx = _half_index(cu_seqlens, 1, lse.shape[1]).to(lse.device)
    lse[:, idx] = torch.logaddexp(lse[:, idx], lse_per_step)


def thd_read_second_half_lse(lse: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    if _cuda(lse):
        return _ext.get().thd_read_second_half_lse(lse.contiguous(), _cu32(cu_seqlens, lse.device))
    return lse[:, _half_index(cu_seqlens, 1, lse.shape[1]).to(lse.device)].contiguous()


def thd_out_correction(out: torch.Tensor, out_per_step: torch.Tensor, lse: torch.Tensor, lse_per_step: torch.Tensor,
                       cu_seqlens: torch.Tensor, only_second_half: bool) -> None:
    """In place: ``out += out_per_step * exp(lse_per_step - lse)`` on all tokens or on the second halves."""
    if _cuda(out, out_per_step, lse, lse_per_step):
        _ext.get().thd_out_correction(out, out_per_step.contiguous(), lse.contiguous(), lse_per_step.contiguous(),
                                      _cu32(cu_seqlens, out.device), only_second_half)
        return
    if only_second_half:
        idx = _half_index(cu_seqlens, 1, out.shape[0]).to(out.device)
        w = torch.nan_to_num(torch.exp(lse_per_step - lse[:, idx]), nan=0.0).t().unsqueeze(-1)
        out[idx] = (out[idx].float() + out_per_step.float() * w).to(out.dtype)
    else:
        w = torch.nan_to_num(torch.exp(lse_per_step - lse), nan=0.0).t().unsqueeze(-1)
        out.copy_((out.float() + out_per_step.float() * w).to(out.dtype))


def thd_grad_correction(grad: torch.Tensor, grad_per_step: torch.Tensor, cu_seqlens: torch.Tensor, first_half: str,
                        second_half: str) -> None:
    """In place, per half of every sequence: ``"none"`` leaves ``grad``, ``"copy"`` overwrites it with
    ``grad_per_step``, ``"add"`` accumulates.  ``grad_per_step`` covers all tokens, or only the tokens
    of the single half that is not ``"none"``.  Tensors are ``[t, ...]`` or stacked ``[2, t, ...]``."""
    stacked = grad.dim() == 4
    if _cuda(grad, grad_per_step):
        _ext.get().thd_grad_correction(grad, grad_per_step.contiguous(), _cu32(cu_seqlens, grad.device),
                                       _MODES[first_half], _MODES[second_half], stacked)
        return
    sd = 1 if stacked else 0
    t, ts = grad.shape[sd], grad_per_step.shape[sd]
    cu = cu_seqlens.tolist()
    for half, mode in ((0, first_half), (1, second_half)):
        if mode == "none":
            continue
        idx: List[int] = []
        for a, b in zip(cu[:-1], cu[1:]):
            hl = (b - a) // 2
            idx.extend(range(a + half * hl, a + half * hl + hl))
        dst = torch.tensor(idx, dtype=torch.long, device=grad.device)
        if ts == t:
            src = grad_per_step.index_select(sd, dst)
        else:
            pos = torch.tensor([i for a, b in zip(cu[:-1], cu[1:]) for i in range(a // 2, a // 2 + (b - a) // 2)],
                               dtype=torch.long, device=grad.device)
            src = grad_per_step.index_select(sd, pos)
        cur = grad.index_select(sd, dst)
        grad.index_copy_(sd, dst, src if mode == "copy" else (cur.float() + src.float()).to(grad.dtype))


def convert_thd_to_bshd(tensor: torch.Tensor, cu_seqlens: torch.Tensor, b: int, max_seq_len: int) -> torch.Tensor:
    """``[t, ...]`` -> zero-padded ``[b, max_seq_len, ...]``."""
    if _cuda(tensor) and (tensor[0].numel() * tensor.element_size()) % 16 == 0:
        return _ext.get().convert_thd_to_bshd(tensor, _cu32(cu_seqlens, tensor.device), b, max_seq_len)
    out = tensor.new_zeros(b, max_seq_len, *tensor.shape[1:])
    cu = cu_seqlens.tolist()
    for i, (a, e) in enumerate(zip(cu[:-1], cu[1:])):
        n = min(e - a, max_seq_len)
        out[i, :n] = tensor[a:a + n]
    return out


def convert_bshd_to_thd(tensor: torch.Tensor, cu_seqlens: torch.Tensor, t: int) -> torch.Tensor:
    """``[b, s, ...]`` -> packed ``[t, ...]`` (tokens past the last sequence are zero)."""
    if _cuda(tensor) and (tensor[0, 0].numel() * tensor.element_size()) % 16 == 0:
        return _ext.get().convert_bshd_to_thd(tensor, _cu32(cu_seqlens, tensor.device), t)
    out = tensor.new_zeros(t, *tensor.shape[2:])
    cu = cu_seqlens.tolist()
    for i, (a, e) in enumerate(zip(cu[:-1], cu[1:])):
        n = min(e - a, tensor.shape[1])
        out[a:a + n] = tensor[i, :n]
    return out


def kv_cache_step(new_k: torch.Tensor, new_v: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor,
                  page_table: torch.Tensor, cu_new: torch.Tensor, cu_kv: torch.Tensor,
                  total: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Append every live sequence's new tokens to a paged cache ``[pages, page_size, h, d]`` and return
    all sequences' keys / values (old and new) packed as ``[total, h, d]``.  ``page_table`` is
    ``[sequences, width]`` int32; ``cu_new`` / ``cu_kv`` are the cumulative new / resulting lengths.
    A contiguous cache ``[slots, max_len, h, d]`` is the case width 1, page table = slot per sequence."""
    if _cuda(new_k, new_v, cache_k, cache_v) and \
            (cache_k[0, 0].numel() * cache_k.element_size()) % 16 == 0 and \
            (cache_v[0, 0].numel() * cache_v.element_size()) % 16 == 0:
        C_ = _ext.get()
        dev = cache_k.device
        k, v = C_.kv_cache_step(new_k, new_v, cache_k, cache_v, _cu32(page_table, dev), _cu32(cu_new, dev),
                                _cu32(cu_kv, dev), total, C_.status(dev.index))
        return k, v
    ps = cache_k.shape[1]
    cn, ck, pt = cu_new.tolist(), cu_kv.tolist(), page_table.tolist()
    ks, vs = [], []
    for i in range(len(ck) - 1):
        n, tot = cn[i + 1] - cn[i], ck[i + 1] - ck[i]
        old = tot - n
        pages = torch.tensor(pt[i], dtype=torch.long, device=cache_k.device)
        pos = torch.arange(old, tot, device=cache_k.device)
        cache_k[pages[pos // ps], pos % ps] = new_k[cn[i]:cn[i + 1]]
        cache_v[pages[pos // ps], pos % ps] = new_v[cn[i]:cn[i + 1]]
        allp = torch.arange(tot, device=cache_k.device)
        ks.append(cache_k[pages[allp // ps], allp % ps])
        vs.append(cache_v[pages[allp // ps], allp % ps])
    return torch.cat(ks, dim=0), torch.cat(vs, dim=0)


def _cp_rank_order_index(cu_seqlens: torch.Tensor, total_tokens: int, cp_size: int) -> torch.Tensor:
    """Token indices (sequence order) listed rank by rank: position j of the result is the token that
    sits at position j of the concatenation of all ranks' shards."""
    return torch.cat([thd_get_partitioned_indices(cu_seqlens, total_tokens, cp_size, r).long() for r in range(cp_size)])


def thd_sequence_order_to_cp_rank_order(inp: torch.Tensor, cu_seqlens: torch.Tensor, cp_size: int,
                                        total_tokens: int) -> torch.Tensor:
    """Reorder packed tokens from sequence order to the concatenation of the context-parallel ranks'
    shards (what an all-gather over the group produces)."""
    assert inp.shape[0] == total_tokens and total_tokens % (2 * cp_size) == 0
    return inp.index_select(0, _cp_rank_order_index(cu_seqlens, total_tokens, cp_size).to(inp.device))


def thd_cp_rank_order_to_sequence_order(inp: torch.Tensor, cu_seqlens: torch.Tensor, cp_size: int,
                                        total_tokens: int) -> torch.Tensor:
    """Inverse of :func:`thd_sequence_order_to_cp_rank_order`."""
    assert inp.shape[0] == total_tokens and total_tokens % (2 * cp_size) == 0
    out = torch.empty_like(inp)
    out.index_copy_(0, _cp_rank_order_index(cu_seqlens, total_tokens, cp_size).to(inp.device), inp)
    return out


def thd_reorder_between_sequence_and_cp_rank_order(inp: torch.Tensor, cu_seqlens: torch.Tensor, cp_size: int,
                                                   cp_rank_to_sequence_order: bool, total_tokens: int) -> torch.Tensor:
    fn = thd_cp_rank_order_to_sequence_order if cp_rank_to_sequence_order else thd_sequence_order_to_cp_rank_order
    return fn(inp, cu_seqlens, cp_size, total_tokens)
