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

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


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
                                   expert_bias: Optional[torch.Tensor] = None, routing_map_format: str = "bytemap",
                                   topk_indices: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(probs [T, E] in the dtype of logits, routing_map bool [T, E])``."""
    assert logits.dtype != torch.float64, "float64 router logits are not supported"
    shape = logits.shape
    E = shape[-1]
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
    if routing_map_format in ("bitmap_u8", 1):
        Ep = (E + 7) // 8 * 8
        bits = F.pad(rmap, (0, Ep - E)).reshape(-1, Ep // 8, 8).to(torch.uint8)
        weights = (2 ** torch.arange(8, device=lf.device)).to(torch.uint8)
        rmap = (bits * weights).sum(-1).to(torch.uint8).reshape(*shape[:-1], Ep // 8)
        return probs.to(logits.dtype).reshape(shape), rmap
    return probs.to(logits.dtype).reshape(shape), rmap.reshape(shape)


def fused_compute_score_for_moe_aux_loss(logits: torch.Tensor, topk: int, score_function: str = "softmax"
                                         ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scores used by the auxiliary loss: full score-function output (normalised over experts for
    sigmoid / sqrt-softplus) and the plain top-k routing map.  Returns ``(routing_map, scores)``."""
    E = logits.shape[-1]
    lf = logits.float().reshape(-1, E)
    scores = _score(lf, score_function)
    if score_function != "softmax":
        scores = scores / (scores.sum(-1, keepdim=True) + 1e-20)
    idx = scores.detach().topk(topk, dim=-1).indices
    rmap = torch.zeros(lf.shape, dtype=torch.bool, device=lf.device).scatter_(1, idx, True)
    return rmap.reshape(logits.shape), scores.reshape(logits.shape)


def fused_moe_aux_loss(probs: torch.Tensor, tokens_per_expert: torch.Tensor, total_num_tokens: int,
                       num_experts: int, num_rows: Optional[int] = None, num_cols: Optional[int] = None,
                       topk: int = 1, coeff: float = 0.0) -> torch.Tensor:
    """``coeff * E / (topk * T^2) * sum_e (sum_t probs[t, e]) * tokens_per_expert[e]``."""
    agg = probs.float().reshape(-1, probs.shape[-1]).sum(0)
    c = num_experts * coeff / (topk * float(total_num_tokens) * float(total_num_tokens))
    return (agg * tokens_per_expert.float()).sum() * c
