"""Vocabulary-parallel cross entropy as a public function (reference:
``pytorch/cross_entropy.py`` over Triton kernels; here the fused CUDA kernels of
``csrc/misc/cross_entropy.cu`` and a small all-reduce of per-row statistics)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops
from .models.llama import _FusedCrossEntropy
from .parallel import distributed as D


class _PerTokenCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, group, vocab_start):  # type: ignore[override]
        m, s, t = ops.cross_entropy_stats(logits, labels, vocab_start)
        if group is not None and D.get_world_size(group) > 1:
            gm = m.clone()
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=group)
            st = torch.stack([s * torch.exp(m - gm), t])
            dist.all_reduce(st, group=group)
            gs, gt = st[0], st[1]
        else:
            gm, gs, gt = m, s, t
        ctx.save_for_backward(logits, labels, gm, gs)
        ctx.vocab_start = vocab_start
        return torch.where(labels.reshape(-1) == -100, torch.zeros_like(gs), gm + torch.log(gs) - gt)

    @staticmethod
    def backward(ctx, go):  # type: ignore[override]
        logits, labels, gm, gs = ctx.saved_tensors
        grad = ops.cross_entropy_parallel_grad(logits, labels, gm, gs, ctx.vocab_start, 1.0, inplace_grad=False)
        return (grad.float() * go.reshape(-1, 1).float()).to(logits.dtype), None, None, None


class _SmoothingTerm(torch.autograd.Function):
    """Per row ``x[target] - mean_i x[i]`` over the FULL vocabulary (0 for ignored rows): what label smoothing adds
    to the plain loss, ``loss_eps = loss + eps * (x[target] - mean x)``.  With a group, two floats per row cross
    it."""

    @staticmethod
    def forward(ctx, logits, labels, group, vocab_start):  # type: ignore[override]
        rows, v_local = logits.shape
        valid = labels != -100
        local = labels - vocab_start
        mine = (local >= 0) & (local < v_local) & valid
        idx = local.clamp(0, v_local - 1)
        xt = torch.gather(logits, 1, idx[:, None]).squeeze(1).float() * mine
        st = torch.stack([xt, logits.float().sum(dim=1)])
        world = D.get_world_size(group) if group is not None else 1
        if world > 1:
            dist.all_reduce(st, group=group)
        ctx.save_for_backward(idx, mine, valid)
        ctx.cfg = (v_local, v_local * world, logits.dtype)
        return (st[0] - st[1] / (v_local * world)) * valid

    @staticmethod
    def backward(ctx, go):  # type: ignore[override]
        idx, mine, valid = ctx.saved_tensors
        v_local, v_total, dtype = ctx.cfg
        go = go.float() * valid
        grad = (-go / v_total)[:, None].expand(-1, v_local).clone()
        grad.scatter_add_(1, idx[:, None], (go * mine)[:, None])
        return grad.to(dtype), None, None, None


def parallel_cross_entropy(inp: torch.Tensor, target: torch.Tensor, label_smoothing: float = 0.0,
                           reduce_loss: bool = False, dist_process_group=None, ignore_idx: int = -100,
                           is_cg_capturable: bool = False, *, _input=None) -> torch.Tensor:
    """Cross entropy of ``inp [..., vocab/tp]`` against ``target [...]``.

    With ``dist_process_group`` the vocabulary dimension is sharded over that group (rank ``r``
    holds entries ``[r*V/tp, (r+1)*V/tp)``) and only three floats per row cross the group.
    Returns the mean over non-ignored tokens when ``reduce_loss``, else the per-token losses.
    ``label_smoothing`` mixes the one-hot target with the uniform distribution over the full vocabulary (the
    definition of ``torch.nn.functional.cross_entropy``); it costs one more pass over the logits.
    ``is_cg_capturable`` needs no special path: forward and backward never synchronise with the host, so the
    function can always be recorded in a CUDA graph.
    """
    if _input is not None:      # older keyword of the reference
        inp = _input
    if not 0.0 <= label_smoothing < 1.0:
        raise ValueError(f"label_smoothing must be in [0, 1), got {label_smoothing}")
    shape = target.shape
    logits = inp.reshape(-1, inp.shape[-1])
    tgt = target.reshape(-1)
    if ignore_idx != -100:
        tgt = torch.where(tgt == ignore_idx, torch.full_like(tgt, -100), tgt)
    tp = D.get_world_size(dist_process_group) if dist_process_group is not None else 1
    vocab_start = D.get_rank(dist_process_group) * logits.shape[-1] if tp > 1 else 0
    if label_smoothing == 0.0:
        if reduce_loss:
            return _FusedCrossEntropy.apply(logits, tgt, dist_process_group, vocab_start)
        return _PerTokenCrossEntropy.apply(logits, tgt, dist_process_group, vocab_start).reshape(shape)
    # the target distribution is (1 - eps) on the label plus eps / V everywhere (V = the full vocabulary):
    # loss = lse - (1 - eps) x[t] - eps * mean(x) = plain loss + eps * (x[t] - mean(x))
    loss = _PerTokenCrossEntropy.apply(logits, tgt, dist_process_group, vocab_start) \
        + label_smoothing * _SmoothingTerm.apply(logits, tgt, dist_process_group, vocab_start)
    if reduce_loss:
        return loss.sum() / (tgt != -100).sum().clamp(min=1)
    return loss.reshape(shape)


CrossEntropyFunction = _PerTokenCrossEntropy   # the reference's name of the per-token autograd function
