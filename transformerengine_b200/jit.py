"""Fused element-wise helpers under the reference's module name (``pytorch/jit.py``).  The reference fuses these
with TorchScript / ``torch.compile``; here they call the library's kernels (or plain PyTorch on CPU), so the
"warm-up" functions have nothing to compile and return at once."""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from . import ops as K


def no_torch_dynamo(recursive: bool = True) -> Callable:
    """Decorator that keeps ``torch.compile`` from tracing into a function (it runs eagerly inside compiled code)."""
    def deco(fn):
        try:
            import torch._dynamo

            return torch._dynamo.disable(fn, recursive=recursive)
        except Exception:  # noqa: BLE001
            return fn
    return deco


def set_jit_fusion_options() -> None:
    """Nothing to configure: no TorchScript fuser is used."""


def jit_fuser(fn: Callable) -> Callable:
    return fn


def bias_gelu_fused(inp: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    x = inp if bias is None or bias.numel() == 0 else inp + bias.to(inp.dtype)
    y, _ = K.activation_fwd(x, "gelu")
    return y.to(inp.dtype)


def gelu_fused_(inp: torch.Tensor) -> torch.Tensor:
    return bias_gelu_fused(inp, None)


def bgrad_dgelu_fused(grad_output: torch.Tensor, inp: torch.Tensor, bias: Optional[torch.Tensor]
                      ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Gradient of ``gelu(inp + bias)`` and the bias gradient (column sums) from one kernel."""
    has_bias = bias is not None and bias.numel() != 0
    x = inp + bias.to(inp.dtype) if has_bias else inp
    dx, _, db = K.activation_bwd(grad_output.contiguous(), x, "gelu", want_dbias=has_bias)
    return dx.to(inp.dtype), (db.to(bias.dtype) if db is not None else None)


def dgelu_fused_(grad_output: torch.Tensor, inp: torch.Tensor) -> torch.Tensor:
    return bgrad_dgelu_fused(grad_output, inp, None)[0]


def l2normalization_fused(x: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().sum(-1, keepdim=True) + eps)).to(x.dtype)


def l2normalization_fwd_fused(x: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    rs = torch.rsqrt(xf.square().sum(-1, keepdim=True) + eps)
    return (xf * rs).to(x.dtype), rs


def l2normalization_backward_fused(grad_output: torch.Tensor, x: torch.Tensor, rsqrt_norm: torch.Tensor, eps: float
                                   ) -> torch.Tensor:
    g, xf = grad_output.float(), x.float()
    dot = (g * xf).sum(-1, keepdim=True)
    return (g * rsqrt_norm - xf * dot * rsqrt_norm.pow(3)).to(x.dtype)


def bias_dropout_add(x: torch.Tensor, bias: torch.Tensor, residual: torch.Tensor, prob: float, training: bool
                     ) -> torch.Tensor:
    out = torch.nn.functional.dropout(x + bias.to(x.dtype) if bias is not None and bias.numel() else x, p=prob,
                                      training=training)
    return residual + out


def get_bias_dropout_add(training: bool) -> Callable:
    return lambda x, bias, residual, prob: bias_dropout_add(x, bias, residual, prob, training)


def bias_dropout_add_fused_train(x, bias, residual, prob):
    return bias_dropout_add(x, bias, residual, prob, True)


def bias_dropout_add_fused_inference(x, bias, residual, prob):
    return bias_dropout_add(x, bias, residual, prob, False)


def _nothing_to_warm_up(*_a, **_k) -> None:
    """The kernels are compiled ahead of time."""


warmup_jit_bias_dropout_add = warmup_jit_bias_dropout_add_all_dtypes = _nothing_to_warm_up
warmup_jit_bias_gelu = warmup_jit_bias_gelu_all_dtypes = _nothing_to_warm_up
warmup_jit_l2normalization = warmup_jit_l2normalization_all_dtypes = _nothing_to_warm_up
