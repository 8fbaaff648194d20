"""Fused Adam / AdamW and SGD over whole parameter groups.

One multi-tensor kernel updates the fp32 master copy, both moments and the
model-dtype parameter in a single pass (reference API:
``pytorch/optimizers/fused_adam.py:36-140``, ``fused_sgd.py``).
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch

from .. import ops
from ..modules.base import bump_weights_epoch
from ..tensor.base import QuantizedTensor


class FusedAdam(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, bias_correction: bool = True, betas=(0.9, 0.999),
                 eps: float = 1e-8, adam_w_mode: bool = True, weight_decay: float = 0.0, amsgrad: bool = False,
                 set_grad_none: bool = True, capturable: bool = False, master_weights: bool = False,
                 master_weight_dtype: torch.dtype = torch.float32, exp_avg_dtype: torch.dtype = torch.float32,
                 exp_avg_sq_dtype: torch.dtype = torch.float32, use_decoupled_grad: bool = False,
                 store_param_remainders: bool = False):
        if amsgrad:
            raise RuntimeError("FusedAdam does not support the AMSGrad variant.")
        assert exp_avg_dtype == exp_avg_sq_dtype, "both moments use one dtype"
        assert exp_avg_dtype in (torch.float32, torch.bfloat16), "moments are fp32 or bf16"
        defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.adam_w_mode = adam_w_mode
        self.set_grad_none = set_grad_none
        self.capturable = capturable
        self.master_weights = master_weights
        self.state_dtype = exp_avg_dtype
        self.use_decoupled_grad = use_decoupled_grad
        self._noop = None

    def zero_grad(self, set_to_none: Optional[bool] = None):  # type: ignore[override]
        set_to_none = self.set_grad_none if set_to_none is None else set_to_none
        for g in self.param_groups:
            for p in g["params"]:
                if self.use_decoupled_grad and hasattr(p, "decoupled_grad"):
                    p.decoupled_grad = None
                if set_to_none:
                    p.grad = None
                elif p.grad is not None:
                    p.grad.zero_()

    def _init_state(self, p):
        st = self.state[p]
        if "exp_avg" not in st:
            base = p.dequantize() if isinstance(p, QuantizedTensor) else p.detach()
            st["exp_avg"] = torch.zeros(base.shape, dtype=self.state_dtype, device=base.device)
            st["exp_avg_sq"] = torch.zeros(base.shape, dtype=self.state_dtype, device=base.device)
            if self.master_weights or isinstance(p, QuantizedTensor):
                hp = getattr(p, "_high_precision_init_val", None)
                st["master_param"] = (hp.to(base.device) if hp is not None else base).float().clone()
        return st

    @torch.no_grad()
    def step(self, closure=None, grad_scaler=None):  # type: ignore[override]
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            if not group["params"]:
                continue
            group["step"] = group.get("step", 0) + 1
            b1, b2 = group["betas"]
            buckets = {}
            quantized = []
            for p in group["params"]:
                g = getattr(p, "decoupled_grad", None) if self.use_decoupled_grad else p.grad
                if g is None:
                    continue
                st = self._init_state(p)
                if isinstance(p, QuantizedTensor):
                    quantized.append((p, g, st))
                    continue
                has_master = "master_param" in st
                key = (g.dtype, p.dtype, has_master)
                b = buckets.setdefault(key, [[], [], [], [], []])
                b[0].append(g)
                b[1].append(p.data)
                b[2].append(st["exp_avg"])
                b[3].append(st["exp_avg_sq"])
                if has_master:
                    b[4].append(st["master_param"])
            for (gd, pd, has_master), lists in buckets.items():
                ls = lists if has_master else lists[:4]
                ops.multi_tensor_adam(ls, group["lr"], b1, b2, group["eps"], group["step"], self.adam_w_mode,
                                      group["bias_correction"], group["weight_decay"])
            for p, g, st in quantized:
                # quantized parameters: update the fp32 master, then re-quantize in place
                tmp = st["master_param"].clone()
                ops.multi_tensor_adam([[g.float()], [tmp], [st["exp_avg"]], [st["exp_avg_sq"]], [st["master_param"]]],
                                      group["lr"], b1, b2, group["eps"], group["step"], self.adam_w_mode,
                                      group["bias_correction"], group["weight_decay"])
                p.quantize_(st["master_param"])
        bump_weights_epoch()
        return loss

    def state_dict(self):  # type: ignore[override]
        sd = super().state_dict()
        for st in sd["state"].values():
            for k in ("exp_avg", "exp_avg_sq"):
                if k in st and st[k].dtype != torch.float32:
                    st[k] = st[k].float()  # checkpoints always hold unscaled fp32 moments
        return sd

    def load_state_dict(self, state_dict):  # type: ignore[override]
        super().load_state_dict(state_dict)
        for st in self.state.values():
            for k in ("exp_avg", "exp_avg_sq"):
                if k in st and st[k].dtype != self.state_dtype:
                    st[k] = st[k].to(self.state_dtype)
            if "master_param" in st:
                st["master_param"] = st["master_param"].float()
        bump_weights_epoch()


class FusedSGD(torch.optim.Optimizer):
    def __init__(self, params, lr: float, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
                 nesterov: bool = False, wd_after_momentum: bool = False, materialize_master_grads: bool = True,
                 set_grad_none: bool = False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov))
        self.wd_after_momentum = wd_after_momentum
        self.set_grad_none = set_grad_none

    @torch.no_grad()
    def step(self, closure=None):  # type: ignore[override]
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            for first in (True, False):
                buckets = {}
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    st = self.state[p]
                    is_first = "momentum_buffer" not in st
                    if is_first != first:
                        continue
                    if is_first:
                        st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                    b = buckets.setdefault((p.grad.dtype, p.dtype), [[], [], []])
                    b[0].append(p.grad)
                    b[1].append(p.data)
                    b[2].append(st["momentum_buffer"])
                for lists in buckets.values():
                    ops.multi_tensor_sgd(lists, group["lr"], group["momentum"], group["dampening"],
                                         group["weight_decay"], group["nesterov"], first, self.wd_after_momentum)
        bump_weights_epoch()
        return loss


def multi_tensor_applier(op, noop_flag, tensor_lists, *args):
    """Reference-style entry: ``op(chunk, noop, lists, *args)``."""
    return op(2048 * 32, noop_flag, tensor_lists, *args)
