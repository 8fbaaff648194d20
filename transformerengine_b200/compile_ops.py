"""The library's kernels as ``torch.library`` custom operators, so that ``torch.compile`` and ``torch.export``
see them as single opaque nodes (with shape / dtype inference and autograd formulas) instead of breaking the
graph at every extension call.

    import transformerengine_b200.compile_ops as cops

    @torch.compile(fullgraph=True)
    def block(x, g, w1, w2):
        h = cops.rmsnorm(x, g, 1e-5)
        return cops.linear(cops.swiglu(cops.linear(h, w1)), w2)

Operators (namespace ``teb200``): ``rmsnorm``, ``layernorm``, ``activation`` (all the library's activations,
gated ones included), ``linear`` (``x W^T (+ b)`` on the tcgen05 GEMM), ``rope``, ``cross_entropy``.  Each runs the
same code path as the eager functional layer (CUDA kernels on a GPU, the PyTorch oracle on CPU); the fake
implementations only compute output shapes.  Quantized (FP8 / MXFP8 / NVFP4) execution keeps using the modules:
their quantizer state lives in Python objects that a traced graph cannot carry.
(Reference: ``pytorch/export.py`` and the ``torch.compile`` notes of ``pytorch/jit.py``; the operator set and the
registration code are this library's own.)
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch.library import custom_op

from . import ops as K

_GATED = ("swiglu", "geglu", "reglu", "qgeglu", "sreglu")


# ------------------------------------------------------------------------------------------------- norms
@custom_op("teb200::norm_fwd", mutates_args=())
def _norm_fwd(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float, zero_centered: bool,
              layernorm: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    y, _, mu, rs = K.norm_fwd(x, gamma, beta, eps, zero_centered, layernorm)
    if mu is None:
        mu = rs.new_empty(0)
    return y, mu, rs


@_norm_fwd.register_fake
def _(x, gamma, beta, eps, zero_centered, layernorm):
    rows = x.numel() // x.shape[-1]
    rs = x.new_empty(rows, dtype=torch.float32)
    return torch.empty_like(x), (x.new_empty(rows, dtype=torch.float32) if layernorm else x.new_empty(0, dtype=torch.float32)), rs


@custom_op("teb200::norm_bwd", mutates_args=())
def _norm_bwd(dy: torch.Tensor, x: torch.Tensor, mu: torch.Tensor, rs: torch.Tensor, gamma: torch.Tensor,
              zero_centered: bool, layernorm: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dx, dg, db = K.norm_bwd(dy.contiguous(), x, mu if layernorm else None, rs, gamma, zero_centered, layernorm)
    if db is None:
        db = dg.new_empty(0)
    return dx, dg, db


@_norm_bwd.register_fake
def _(dy, x, mu, rs, gamma, zero_centered, layernorm):
    return torch.empty_like(x), torch.empty_like(gamma), (torch.empty_like(gamma) if layernorm else gamma.new_empty(0))


def _norm_setup(ctx, inputs, output):
    x, gamma, beta, eps, zero_centered, layernorm = inputs
    _, mu, rs = output
    ctx.save_for_backward(x, gamma, mu, rs)
    ctx.cfg = (zero_centered, layernorm, beta is not None)


def _norm_backward(ctx, dy, dmu, drs):
    x, gamma, mu, rs = ctx.saved_tensors
    zc, ln, has_beta = ctx.cfg
    dx, dg, db = _norm_bwd(dy, x, mu, rs, gamma, zc, ln)
    return dx, dg, (db if has_beta else None), None, None, None


_norm_fwd.register_autograd(_norm_backward, setup_context=_norm_setup)


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-5, zero_centered_gamma: bool = False) -> torch.Tensor:
    return _norm_fwd(x, gamma, None, eps, zero_centered_gamma, False)[0]


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5,
              zero_centered_gamma: bool = False) -> torch.Tensor:
    return _norm_fwd(x, gamma, beta, eps, zero_centered_gamma, True)[0]


# ------------------------------------------------------------------------------------------- activations
@custom_op("teb200::activation_fwd", mutates_args=())
def _act_fwd(x: torch.Tensor, name: str) -> torch.Tensor:
    y, _ = K.activation_fwd(x, name)
    return y.to(x.dtype)


@_act_fwd.register_fake
def _(x, name):
    shape = list(x.shape)
    if name in _GATED:
        shape[-1] //= 2
    return x.new_empty(shape)


@custom_op("teb200::activation_bwd", mutates_args=())
def _act_bwd(dy: torch.Tensor, x: torch.Tensor, name: str) -> torch.Tensor:
    dx, _, _ = K.activation_bwd(dy.contiguous(), x, name)
    return dx.to(x.dtype)


@_act_bwd.register_fake
def _(dy, x, name):
    return torch.empty_like(x)


def _act_setup(ctx, inputs, output):
    x, name = inputs
    ctx.save_for_backward(x)
    ctx.name = name


def _act_backward(ctx, dy):
    (x,) = ctx.saved_tensors
    return _act_bwd(dy, x, ctx.name), None


_act_fwd.register_autograd(_act_backward, setup_context=_act_setup)


def activation(x: torch.Tensor, name: str) -> torch.Tensor:
    """``name``: gelu, relu, silu, qgelu, srelu, swiglu, geglu, reglu, ... (gated ones halve the last dimension)."""
    return _act_fwd(x, name)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    return _act_fwd(x, "swiglu")


# -------------------------------------------------------------------------------------------------- GEMM
@custom_op("teb200::gemm_nt", mutates_args=())
def _gemm_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T (+ bias [N])``"""
    return K.gemm_nt(a.contiguous(), b.contiguous(), out_dtype=a.dtype, bias=bias)


@_gemm_nt.register_fake
def _(a, b, bias):
    return a.new_empty(a.shape[0], b.shape[0])


def _gemm_setup(ctx, inputs, output):
    a, b, bias = inputs
    ctx.save_for_backward(a, b)
    ctx.has_bias = bias is not None
    ctx.bias_dtype = bias.dtype if bias is not None else None


def _gemm_backward(ctx, dy):
    a, b = ctx.saved_tensors
    dy = dy.contiguous()
    da = _gemm_nt(dy, b.t(), None) if ctx.needs_input_grad[0] else None          # dy [M, N] @ b [N, K]
    db = _gemm_nt(dy.t(), a.t(), None) if ctx.needs_input_grad[1] else None      # dy^T [N, M] @ a [M, K]
    dbias = K.column_sum(dy, ctx.bias_dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
    return da, db, dbias


_gemm_nt.register_autograd(_gemm_backward, setup_context=_gemm_setup)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [..., K] @ weight [N, K]^T (+ bias)`` on the library's GEMM."""
    lead = x.shape[:-1]
    y = _gemm_nt(x.reshape(-1, x.shape[-1]), weight, bias)
    return y.reshape(*lead, weight.shape[0])


# -------------------------------------------------------------------------------------------------- RoPE
@custom_op("teb200::rope", mutates_args=())
def _rope(x: torch.Tensor, freqs: torch.Tensor, interleaved: bool, backward: bool) -> torch.Tensor:
    return K.rope_apply(x.contiguous(), freqs, interleaved=interleaved, backward=backward)


@_rope.register_fake
def _(x, freqs, interleaved, backward):
    return torch.empty_like(x)


def _rope_setup(ctx, inputs, output):
    _, freqs, interleaved, backward = inputs
    ctx.save_for_backward(freqs)
    ctx.cfg = (interleaved, backward)


def _rope_backward(ctx, dy):
    (freqs,) = ctx.saved_tensors
    interleaved, backward = ctx.cfg
    return _rope(dy, freqs, interleaved, not backward), None, None, None


_rope.register_autograd(_rope_backward, setup_context=_rope_setup)


def rope(x_sbhd: torch.Tensor, freqs: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """Rotary embedding of ``[s, b, h, d]`` with the angle table ``[s, d_rot]`` (or ``[s, 1, 1, d_rot]``)."""
    return _rope(x_sbhd, freqs.reshape(freqs.shape[0], freqs.shape[-1]).float(), interleaved, False)


# --------------------------------------------------------------------------------------- cross entropy
@custom_op("teb200::cross_entropy", mutates_args=())
def _cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row loss and d(sum of losses)/d(logits) from one pass over the logits."""
    loss, grad = K.cross_entropy_fwd_bwd(logits.contiguous(), targets, 1.0, 0.0, ignore_index, inplace_grad=False)
    return loss, grad


@_cross_entropy.register_fake
def _(logits, targets, ignore_index):
    rows = logits.numel() // logits.shape[-1]
    return logits.new_empty(rows, dtype=torch.float32), torch.empty_like(logits)


def _ce_setup(ctx, inputs, output):
    ctx.save_for_backward(output[1])


def _ce_backward(ctx, dloss, dgrad):
    (g,) = ctx.saved_tensors
    return (g.reshape(-1, g.shape[-1]) * dloss.reshape(-1, 1).to(g.dtype)).reshape(g.shape), None, None


_cross_entropy.register_autograd(_ce_backward, setup_context=_ce_setup)


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Per-row cross entropy (fp32, shape of ``targets``); the gradient is produced in the forward pass."""
    loss, _ = _cross_entropy(logits, targets, ignore_index)
    return loss.reshape(targets.shape)


__all__: List[str] = ["rmsnorm", "layernorm", "activation", "swiglu", "linear", "rope", "cross_entropy"]
