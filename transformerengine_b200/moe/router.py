"""MoE router: score function + top-k (+ group-limited routing, expert bias, scaling) and the
load-balancing auxiliary loss.

Semantics follow the reference kernels (``common/fused_router/
fused_topk_with_score_function.cu:107-300``, ``fused_moe_aux_loss.cu:21-107``): logits are
promoted to fp32; ``expert_bias`` influences only which experts are selected; sigmoid /
sqrt-softplus scores of the chosen experts are renormalised when ``topk > 1``; ``probs`` is a
dense ``[T, E]`` tensor that is zero outside the top-k; the routing map is a bool map.
Everything is differentiable through ``probs``.
"""
from __future__ import annotations

import enum
import math
from typing import Optional, Tuple, Union

import torch
import torch.nn.functional as F


class RoutingMapFormat(enum.IntEnum):
    """Layout of the routing map: ``BYTEMAP`` bool ``[T, E]``; ``BITMAP_U8`` uint8 ``[T, ceil(E / 8)]`` with bit
    ``e % 8`` of byte ``e // 8`` set when the token goes to expert ``e``."""
    BYTEMAP = 0
    BITMAP_U8 = 1


class QBHistogramMode(enum.IntEnum):
    """How the reference builds the quantile-balancing histogram (a second kernel, or atomics inside the router
    kernel).  Both give the same histogram; the names are accepted for compatibility."""
    TWO_KERNEL = 0
    FUSED_ATOMIC = 1


def _map_format(fmt: Union[str, int, RoutingMapFormat]) -> int:
    if isinstance(fmt, str):
        if fmt not in ("bytemap", "bitmap_u8"):
            raise ValueError(f"routing_map_format string must be 'bytemap' or 'bitmap_u8', got {fmt!r}")
        return int(fmt == "bitmap_u8")
    if isinstance(fmt, int) and int(fmt) in (0, 1):
        return int(fmt)
    raise ValueError(f"routing_map_format must be 'bytemap' / 'bitmap_u8', a RoutingMapFormat or 0 / 1; got {fmt!r}")


def _pack_bitmap(rmap: torch.Tensor) -> torch.Tensor:
    """bool ``[T, E]`` -> uint8 ``[T, ceil(E / 8)]``, least significant bit first."""
    T, E = rmap.shape
    Ep = (E + 7) // 8 * 8
    bits = F.pad(rmap, (0, Ep - E)).reshape(T, Ep // 8, 8).to(torch.uint8)
    weights = (2 ** torch.arange(8, device=rmap.device)).to(torch.uint8)
    return (bits * weights).sum(-1).to(torch.uint8)


def _check_bin_bounds(bounds: torch.Tensor) -> Tuple[float, float]:
    """``[lower, upper]`` of the histogram bins, read on the host once per version of the tensor."""
    if not (isinstance(bounds, torch.Tensor) and bounds.dtype == torch.float32 and tuple(bounds.shape) == (2,)):
        raise ValueError("qb_bin_bounds must be a float32 tensor [lower, upper]")
    cached = getattr(bounds, "_qb_checked", None)
    if cached is not None and cached[0] == bounds._version:
        return cached[1]
    if bounds.is_cuda and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("qb_bin_bounds must be validated by an eager router call before CUDA graph capture")
    lower, upper = bounds.detach().cpu().tolist()
    if not (math.isfinite(lower) and math.isfinite(upper) and lower < upper):
        raise ValueError(f"qb_bin_bounds must be finite with lower < upper, got [{lower}, {upper}]")
    bounds._qb_checked = (bounds._version, (lower, upper))
    return lower, upper


def _score(logits: torch.Tensor, score_function: str) -> torch.Tensor:
    if score_function == "softmax":
        return torch.softmax(logits, dim=-1)
    if score_function == "sigmoid":
        return torch.sigmoid(logits)
    if score_function == "sqrtsoftplus":
        return torch.sqrt(F.softplus(logits))
    raise ValueError(f"unsupported score function {score_function}")


def _group_limited_mask(scores: torch.Tensor, topk: int, num_groups: int, group_topk: int) -> torch.Tensor:
    """True where an expert belongs to one of the ``group_topk`` best groups of its token; a
    group's score is the sum of its top ``topk // group_topk`` experts."""
    T, E = scores.shape
    g = scores.reshape(T, num_groups, E // num_groups)
    per = max(topk // group_topk, 1)
    gscore = g.topk(per, dim=-1).values.sum(-1)
    keep = torch.zeros_like(gscore, dtype=torch.bool)
    keep.scatter_(1, gscore.topk(group_topk, dim=-1).indices, True)
    return keep[:, :, None].expand_as(g).reshape(T, E)


_SCORE_FN = {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}


class _RouterTopK(torch.autograd.Function):
    """CUDA fast path: one warp per token computes scores, top-k, probabilities and the map."""

    @staticmethod
    def forward(ctx, logits2d, topk, pre_softmax, scaling, fn, bias):  # type: ignore[override]
        from ..ops import _ext

        C_ = _ext.get()
        probs, rmap, _, _, _ = C_.router_topk(logits2d, topk, pre_softmax, scaling, fn,
                                              None if bias is None else bias.float().contiguous(), False)
        ctx.save_for_backward(logits2d, rmap)
        ctx.cfg = (topk, pre_softmax, scaling, fn)
        ctx.mark_non_differentiable(rmap)
        return probs.to(logits2d.dtype), rmap

    @staticmethod
    def backward(ctx, gprobs, _gmap):  # type: ignore[override]
        from ..ops import _ext

        logits2d, rmap = ctx.saved_tensors
        topk, pre, scaling, fn = ctx.cfg
        g = _ext.get().router_topk_bwd(logits2d, rmap, gprobs.float().contiguous(), topk, pre, scaling, fn)
        return g, None, None, None, None, None


def _cuda_router_ok(logits, topk, num_groups, group_topk, routing_map_format, topk_indices) -> bool:
    from ..ops import _ext

    return (_ext.use_cuda(logits) and hasattr(_ext.get(), "router_topk") and logits.shape[-1] <= 256 and 1 <= topk <= 8
            and not (num_groups is not None and group_topk is not None and num_groups > 1)
            and routing_map_format == "bytemap" and topk_indices is None
            and logits.dtype in (torch.float32, torch.bfloat16, torch.float16))


def fused_topk_with_score_function(logits: torch.Tensor, topk: int, use_pre_softmax: bool = False,
                                   num_groups: Optional[int] = None, group_topk: Optional[int] = None,
                                   scaling_factor: Optional[float] = None, score_function: str = "softmax",
                                   expert_bias: Optional[torch.Tensor] = None,
                                   routing_map_format: Union[str, int, RoutingMapFormat] = "bytemap",
                                   topk_indices: Optional[torch.Tensor] = None,
                                   qb_histogram: Optional[torch.Tensor] = None,
                                   qb_bin_bounds: Optional[torch.Tensor] = None,
                                   qb_histogram_mode: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(probs [T, E] in the dtype of logits, routing_map)``; the map is bool ``[T, E]``, bit-packed uint8
    with ``routing_map_format="bitmap_u8"``, or the dense indices when ``topk_indices`` (an output buffer
    ``[T, topk]``) is given.

    Quantile balancing (``qb_histogram`` int32 ``[E, bins]``, ``qb_bin_bounds`` fp32 ``[lower, upper]``,
    ``qb_histogram_mode``; sigmoid scores with ``expert_bias`` only): besides routing, every (token, expert) pair
    adds one count to ``qb_histogram[e, bin]`` where the binned value is ``cutoff_t - sigmoid(logit_te)``, the
    bias expert ``e`` would have needed to enter token ``t``'s top-k (``cutoff_t``: the (k+1)-th largest biased
    score of the token); ``bins`` uniform bins span ``[lower, upper)``, values outside go to the end bins.  The
    caller turns the histogram into per-expert bias updates (a quantile per expert).
    (Reference: ``common/fused_router/fused_topk_with_score_function.cu``, the QB epilogue.)"""
    if logits.dtype == torch.float64:
        raise ValueError("float64 router logits are not supported")
    routing_map_format = "bitmap_u8" if _map_format(routing_map_format) else "bytemap"
    shape = logits.shape
    E = shape[-1]
    qb = (qb_histogram, qb_bin_bounds, qb_histogram_mode)
    if any(a is not None for a in qb):
        if any(a is None for a in qb):
            raise ValueError("qb_histogram, qb_bin_bounds and qb_histogram_mode must be provided together")
        if score_function != "sigmoid":
            raise ValueError("quantile balancing only supports score_function='sigmoid'")
        if expert_bias is None:
            raise ValueError("quantile balancing requires expert_bias")
        if num_groups is not None or group_topk is not None:
            raise ValueError("quantile balancing does not support grouped top-k")
        if qb_histogram_mode not in ("two_kernel", "fused_atomic"):
            raise ValueError(f"qb_histogram_mode must be 'two_kernel' or 'fused_atomic', got {qb_histogram_mode!r}")
        return _route_with_qb_histogram(logits, topk, scaling_factor, expert_bias, routing_map_format, topk_indices,
                                        qb_histogram, qb_bin_bounds)
    if _cuda_router_ok(logits, topk, num_groups, group_topk, routing_map_format, topk_indices):
        probs, rmap = _RouterTopK.apply(logits.reshape(-1, E).contiguous(), topk, bool(use_pre_softmax),
                                        float(scaling_factor) if scaling_factor else 1.0, _SCORE_FN[score_function],
                                        expert_bias)
        return probs.reshape(shape), rmap.bool().reshape(shape)
    lf = logits.float().reshape(-1, E)
    if score_function == "softmax":
        if use_pre_softmax:
            scores = torch.softmax(lf, dim=-1)
            sel = scores
        else:
            scores = None
            sel = lf
    else:
        scores = _score(lf, score_function)
        sel = scores + expert_bias.float() if expert_bias is not None else scores
    if num_groups is not None and group_topk is not None and num_groups > 1:
        mask = _group_limited_mask(sel.detach(), topk, num_groups, group_topk)
        sel = sel.masked_fill(~mask, float("-inf"))
    idx = sel.detach().topk(topk, dim=-1).indices  # selection is not differentiated
    if score_function == "softmax":
        if use_pre_softmax:
            vals = scores.gather(1, idx)
        else:
            vals = torch.softmax(lf.gather(1, idx), dim=-1)
    else:
        vals = scores.gather(1, idx)  # bias is removed again: the kept values are the raw scores
        if topk > 1:
            vals = vals / (vals.sum(-1, keepdim=True) + 1e-20)
    if scaling_factor:
        vals = vals * scaling_factor
    probs = torch.zeros_like(lf).scatter(1, idx, vals)
    rmap = torch.zeros(lf.shape, dtype=torch.bool, device=lf.device).scatter_(1, idx, True)
    if topk_indices is not None:
        topk_indices.copy_(idx.reshape(topk_indices.shape))
        return probs.to(logits.dtype).reshape(shape), topk_indices
    if routing_map_format == "bitmap_u8":
        return probs.to(logits.dtype).reshape(shape), _pack_bitmap(rmap).reshape(*shape[:-1], -1)
    return probs.to(logits.dtype).reshape(shape), rmap.reshape(shape)


def _route_with_qb_histogram(logits, topk, scaling_factor, expert_bias, routing_map_format, topk_indices, histogram,
                             bin_bounds):
    shape = logits.shape
    E = shape[-1]
    if topk >= E:
        raise ValueError("quantile balancing needs a (topk + 1)-th expert: topk must be smaller than the number of experts")
    if histogram.dtype != torch.int32 or histogram.dim() != 2 or histogram.shape[0] != E:
        raise ValueError(f"qb_histogram must be an int32 tensor [num_experts, num_bins], got {tuple(histogram.shape)}")
    lower, upper = _check_bin_bounds(bin_bounds)
    bins = histogram.shape[1]
    lf = logits.float().reshape(-1, E)
    raw = torch.sigmoid(lf)
    biased = raw.detach() + expert_bias.float()
    vals, idx = biased.topk(topk + 1, dim=-1)        # sorted: the last column is the cutoff
    cutoff, idx = vals[:, topk], idx[:, :topk]
    with torch.no_grad():
        b = torch.floor((cutoff[:, None] - raw.detach() - lower) * (bins / (upper - lower))).clamp_(0, bins - 1).long()
        flat = (torch.arange(E, device=lf.device)[None, :] * bins + b).reshape(-1)
        histogram.view(-1).index_add_(0, flat, torch.ones_like(flat, dtype=torch.int32))
    kept = raw.gather(1, idx)                          # the bias only chooses; the kept values are the raw scores
    if topk > 1:
        kept = kept / (kept.sum(-1, keepdim=True) + 1e-20)
    if scaling_factor:
        kept = kept * scaling_factor
    probs = torch.zeros_like(lf).scatter(1, idx, kept).to(logits.dtype).reshape(shape)
    if topk_indices is not None:
        topk_indices.copy_(idx.reshape(topk_indices.shape))
        return probs, topk_indices
    rmap = torch.zeros(lf.shape, dtype=torch.bool, device=lf.device).scatter_(1, idx, True)
    if routing_map_format == "bitmap_u8":
        return probs, _pack_bitmap(rmap).reshape(*shape[:-1], -1)
    return probs, rmap.reshape(shape)


def fused_compute_score_for_moe_aux_loss(logits: torch.Tensor, topk: int, score_function: str = "softmax",
                                         routing_map_format: Union[str, int, RoutingMapFormat] = "bytemap"
                                         ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scores used by the auxiliary loss: full score-function output (normalised over experts for
    sigmoid / sqrt-softplus) and the plain top-k routing map.  Returns ``(routing_map, scores)``."""
    packed = _map_format(routing_map_format) == 1
    E = logits.shape[-1]
    lf = logits.float().reshape(-1, E)
    scores = _score(lf, score_function)
    if score_function != "softmax":
        scores = scores / (scores.sum(-1, keepdim=True) + 1e-20)
    idx = scores.detach().topk(topk, dim=-1).indices
    rmap = torch.zeros(lf.shape, dtype=torch.bool, device=lf.device).scatter_(1, idx, True)
    if packed:
        return _pack_bitmap(rmap).reshape(*logits.shape[:-1], -1), scores.reshape(logits.shape)
    return rmap.reshape(logits.shape), scores.reshape(logits.shape)


def fused_moe_aux_loss(probs: torch.Tensor, tokens_per_expert: torch.Tensor, total_num_tokens: int,
                       num_experts: int, num_rows: Optional[int] = None, num_cols: Optional[int] = None,
                       topk: int = 1, coeff: float = 0.0) -> torch.Tensor:
    """``coeff * E / (topk * T^2) * sum_e (sum_t probs[t, e]) * tokens_per_expert[e]``."""
    agg = probs.float().reshape(-1, probs.shape[-1]).sum(0)
    c = num_experts * coeff / (topk * float(total_num_tokens) * float(total_num_tokens))
    return (agg * tokens_per_expert.float()).sum() * c
