"""Token permutation for MoE: group the (token, expert) pairs expert-major, and the inverse
with probability-weighted merging (reference API: ``pytorch/permutation.py:876-1340``).

The map returned by ``moe_permute`` is ``dest_row`` (int32): ``[T, E]`` for a mask routing map,
``[T, topk]`` for an index map; entry = row of the permuted buffer, or -1.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _dest_rows_from_mask(routing_map: torch.Tensor, align: int = 1):
    """Expert-major stable ordering.  Returns (dest_row [T,E] int64 (-1 = not routed),
    tokens_per_expert [E], padded offsets [E+1])."""
    m = routing_map.bool()
    T, E = m.shape
    counts = m.sum(0)
    padded = (counts + align - 1) // align * align if align > 1 else counts
    offs = torch.zeros(E + 1, dtype=torch.int64, device=m.device)
    offs[1:] = padded.cumsum(0)
    # rank of the token inside its expert: scan the inner dim of the transposed mask (the scan over
    # the outer dim of [T, E] is orders of magnitude slower on the GPU)
    within = (m.t().contiguous().cumsum(1) - 1).t()
    dest = torch.where(m, within + offs[:-1][None, :], torch.full_like(within, -1))
    return dest, counts, offs


class _PermuteRows(torch.autograd.Function):
    """CUDA row scatter ``out[dest[t, s]] = inp[t]`` (zero rows where nothing lands)."""

    @staticmethod
    def forward(ctx, inp, dest, probs, n_out):  # type: ignore[override]
        from ..ops import _ext

        out, pp = _ext.get().permute_rows(inp.contiguous(), dest, None if probs is None else probs.float().contiguous(),
                                          n_out)
        ctx.save_for_backward(dest)
        ctx.has_probs = probs is not None
        ctx.pdtype = probs.dtype if probs is not None else None
        return out, (pp.to(probs.dtype) if probs is not None else None)

    @staticmethod
    def backward(ctx, gout, gpp):  # type: ignore[override]
        from ..ops import _ext

        (dest,) = ctx.saved_tensors
        ginp = _ext.get().unpermute_rows(gout.contiguous(), dest, None)
        gprobs = None
        if ctx.has_probs and gpp is not None:
            d = dest.long()
            gprobs = torch.where(d >= 0, gpp.float()[d.clamp(min=0)], torch.zeros((), device=gpp.device)).to(ctx.pdtype)
        return ginp, None, gprobs, None


class _UnpermuteRows(torch.autograd.Function):
    """CUDA weighted gather ``out[t] = sum_s w[t, s] * inp[dest[t, s]]``."""

    @staticmethod
    def forward(ctx, inp, dest, w):  # type: ignore[override]
        from ..ops import _ext

        wf = None if w is None else w.float().contiguous()
        out = _ext.get().unpermute_rows(inp.contiguous(), dest, wf)
        ctx.save_for_backward(inp, dest, wf if wf is not None else torch.empty(0, device=inp.device))
        ctx.has_w = w is not None
        ctx.wdtype = w.dtype if w is not None else None
        return out

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        from ..ops import _ext

        inp, dest, wf = ctx.saved_tensors
        g = g.contiguous()
        ginp, pp = _ext.get().permute_rows(g, dest, wf if ctx.has_w else None, inp.shape[0])
        gw = None
        if ctx.has_w:
            ginp = (ginp.float() * pp[:, None]).to(inp.dtype)
            d = dest.long()
            valid = d >= 0
            tok = torch.arange(d.shape[0], device=g.device)[:, None].expand_as(d)[valid]
            dots = (inp[d[valid]].float() * g[tok].float()).sum(-1)
            gw = torch.zeros(d.shape, dtype=torch.float32, device=g.device)
            gw[valid] = dots
            gw = gw.to(ctx.wdtype)
        return ginp, None, gw


def _cuda_rows_ok(t: torch.Tensor) -> bool:
    from ..ops import _ext

    return (_ext.use_cuda(t) and hasattr(_ext.get(), "permute_rows") and t.dim() == 2
            and t.dtype in (torch.float32, torch.bfloat16, torch.float16)
            and (t.shape[1] * t.element_size()) % 16 == 0 and t.shape[1] % 2 == 0)


def moe_permute(inp: torch.Tensor, routing_map: torch.Tensor, num_out_tokens: int = 0, max_token_num: int = -1,
                map_type: str = "mask") -> Tuple[torch.Tensor, torch.Tensor]:
    out, _, row_id_map = _permute(inp, routing_map, None, num_out_tokens, map_type, 1)
    return out, row_id_map


def moe_permute_with_probs(inp: torch.Tensor, probs: torch.Tensor, routing_map: torch.Tensor,
                           num_out_tokens: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Also permutes ``probs`` ([T, E]) into a vector aligned with the permuted rows."""
    out, pp, row_id_map = _permute(inp, routing_map, probs, num_out_tokens, "mask", 1)
    return out, pp, row_id_map


def moe_permute_and_pad_with_probs(inp: torch.Tensor, probs: Optional[torch.Tensor], routing_map: torch.Tensor,
                                   tokens_per_expert: torch.Tensor, align_size: int):
    """Permute and pad every expert slab to a multiple of ``align_size`` rows (zero rows).
    Returns (output, permuted_probs, row_id_map, pad_offsets, padded tokens_per_expert)."""
    out, pp, row_id_map = _permute(inp, routing_map, probs, 0, "mask", align_size)
    counts = routing_map.bool().sum(0)
    padded = (counts + align_size - 1) // align_size * align_size
    pad_offsets = torch.zeros_like(padded)
    pad_offsets[1:] = (padded - counts).cumsum(0)[:-1]
    return out, pp, row_id_map, pad_offsets, padded


def _permute(inp, routing_map, probs, num_out_tokens, map_type, align):
    T, H = inp.shape
    if map_type == "index":
        idx = routing_map.long()
        topk = idx.shape[1]
        E = int(idx.max().item()) + 1 if idx.numel() else 1
        flat_e = idx.reshape(-1)
        order = torch.sort(flat_e, stable=True).indices  # expert-major, token order kept
        dest_flat = torch.empty_like(order)
        dest_flat[order] = torch.arange(order.numel(), device=inp.device)
        dest = dest_flat.reshape(T, topk)
        n_out = T * topk
        if num_out_tokens and num_out_tokens < n_out:  # capacity drop: rows beyond num_out_tokens vanish
            dest = torch.where(dest < num_out_tokens, dest, torch.full_like(dest, -1))
            n_out = num_out_tokens
    else:
        dest, counts, offs = _dest_rows_from_mask(routing_map, align)
        n_out = int(offs[-1].item()) if align > 1 or not num_out_tokens else num_out_tokens
        if align == 1 and num_out_tokens:
            dest = torch.where(dest < num_out_tokens, dest, torch.full_like(dest, -1))
    valid = dest >= 0
    tok = torch.arange(T, device=inp.device)[:, None].expand_as(dest)[valid]
    rows = dest[valid]
    from ..tensor.base import QuantizedTensorStorage

    src = inp.dequantize() if isinstance(inp, QuantizedTensorStorage) else inp
    if _cuda_rows_ok(src) and (probs is None or probs.shape == dest.shape):
        out, pp = _PermuteRows.apply(src, dest.to(torch.int32).contiguous(), probs, n_out)
        return out, pp, dest.to(torch.int32)
    out = torch.zeros(n_out, H, dtype=src.dtype, device=src.device).index_put((rows,), src[tok])
    pp = None
    if probs is not None:
        pp = torch.zeros(n_out, dtype=probs.dtype, device=probs.device).index_put((rows,), probs[valid])
    return out, pp, dest.to(torch.int32)


def moe_unpermute(inp: torch.Tensor, row_id_map: torch.Tensor, merging_probs: Optional[torch.Tensor] = None,
                  restore_shape: Optional[torch.Size] = None, map_type: str = "mask",
                  probs: Optional[torch.Tensor] = None, pad_offsets: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum_slots w[t, slot] * inp[dest_row[t, slot]]`` (plain sum without weights)."""
    if merging_probs is None:
        merging_probs = probs
    if _cuda_rows_ok(inp) and (merging_probs is None or merging_probs.shape == row_id_map.shape):
        out = _UnpermuteRows.apply(inp, row_id_map.to(torch.int32).contiguous(), merging_probs)
        return out.reshape(restore_shape) if restore_shape is not None else out
    dest = row_id_map.long()
    T = dest.shape[0]
    H = inp.shape[-1]
    valid = dest >= 0
    tok = torch.arange(T, device=inp.device)[:, None].expand_as(dest)[valid]
    rows = dest[valid]
    vals = inp[rows]
    if merging_probs is not None:
        vals = vals.float() * merging_probs.float()[valid][:, None]
    out = torch.zeros(T, H, dtype=vals.dtype, device=inp.device).index_add(0, tok, vals)
    out = out.to(inp.dtype)
    if restore_shape is not None:
        out = out.reshape(restore_shape)
    return out


def _chunk_sort_rows(n_rows: int, split_sizes: torch.Tensor, sorted_index: torch.Tensor) -> torch.Tensor:
    """Source row of every output row when the chunks of ``split_sizes`` rows are reordered by ``sorted_index``;
    computed on the device of ``split_sizes`` without reading the sizes back to the host."""
    sizes = split_sizes.to(torch.int64)
    idx = sorted_index.to(torch.int64)
    start = torch.cumsum(sizes, 0) - sizes                 # first input row of every chunk
    out_sizes = sizes[idx]
    out_end = torch.cumsum(out_sizes, 0)                   # one past the last output row of every output chunk
    rows = torch.arange(n_rows, device=sizes.device)
    chunk = torch.searchsorted(out_end, rows, right=True).clamp_(max=idx.numel() - 1)
    return start[idx][chunk] + (rows - (out_end - out_sizes)[chunk])


def moe_sort_chunks_by_index(inp: torch.Tensor, split_sizes: torch.Tensor, sorted_index: torch.Tensor) -> torch.Tensor:
    """Split ``inp`` into consecutive chunks of ``split_sizes`` rows and concatenate them in the
    order given by ``sorted_index`` (expert-parallel token exchange).  One gather, no host synchronisation:
    the split sizes stay on the device (they must add up to the number of rows)."""
    src = _chunk_sort_rows(inp.shape[0], split_sizes.to(inp.device), sorted_index.to(inp.device))
    return inp.index_select(0, src)


def moe_sort_chunks_by_index_with_probs(inp, probs, split_sizes, sorted_index):
    out = moe_sort_chunks_by_index(inp, split_sizes, sorted_index)
    pr = moe_sort_chunks_by_index(probs.reshape(-1, 1), split_sizes, sorted_index).reshape(-1)
    return out, pr
