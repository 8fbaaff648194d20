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


def _local(t):
    """The shard this rank owns when ``t`` is a ``DTensor`` (FSDP2 ``fully_shard`` parameters and their gradients):
    the optimizer state is kept for, and the kernels run on, the local shard; plain tensors pass through."""
    loc = getattr(t, "_local_tensor", None)
    return loc if loc is not None else t


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
        if store_param_remainders and not master_weights:
            raise RuntimeError("store_param_remainders splits the fp32 master weights; it needs master_weights=True")
        if master_weight_dtype != torch.float32:
            raise NotImplementedError("master weights are kept in fp32 (or as bf16 + 16-bit remainders)")
        self.adam_w_mode = adam_w_mode
        self.set_grad_none = set_grad_none
        # capturable: the step count (and a tensor learning rate) stay on the device, so ``step()`` issues
        # the same launches every time and can be recorded in a CUDA graph
        self.capturable = capturable
        self.master_weights = master_weights
        self.store_param_remainders = store_param_remainders
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

    def _init_state(self, key, p):
        """``key`` is the parameter the optimizer was given, ``p`` its local data (the same object unless the
        parameter is a sharded ``DTensor``)."""
        st = self.state[key]
        if "exp_avg" not in st:
            base = p.dequantize() if isinstance(p, QuantizedTensor) else p.detach()
            st["exp_avg"] = torch.zeros(base.shape, dtype=self.state_dtype, device=base.device)
            st["exp_avg_sq"] = torch.zeros(base.shape, dtype=self.state_dtype, device=base.device)
            if self.master_weights or isinstance(p, QuantizedTensor):
                hp = getattr(p, "_high_precision_init_val", None)
                master = (hp.to(base.device) if hp is not None else base).float().clone()
                if self.store_param_remainders and p.dtype == torch.bfloat16 and not isinstance(p, QuantizedTensor):
                    # the bf16 parameter already is the high half of the master weight: keep only the low half
                    hi, lo = ops.misc.split_param_remainder(master)
                    p.data.copy_(hi)
                    st["param_remainder"] = lo
                else:
                    st["master_param"] = master
        return st

    def _step_value(self, group):
        """Host int, or (capturable) an int32 device scalar advanced by a device op."""
        if not self.capturable:
            group["step"] = group.get("step", 0) + 1
            return group["step"]
        st = group.get("step")
        if not isinstance(st, torch.Tensor):
            dev = next((p.device for p in group["params"]), torch.device("cpu"))
            st = group["step"] = torch.full((), int(st or 0), dtype=torch.int32, device=dev)
        st += 1
        return st

    def _lr_value(self, group):
        lr = group["lr"]
        if self.capturable and not isinstance(lr, torch.Tensor):
            cache = group.get("_lr_dev")
            if cache is None or cache[0] != lr:
                dev = next((p.device for p in group["params"]), torch.device("cpu"))
                cache = group["_lr_dev"] = (lr, torch.full((), float(lr), dtype=torch.float32, device=dev))
            return cache[1]
        return lr

    @torch.no_grad()
    def step(self, closure=None, grad_scaler=None):  # type: ignore[override]
        if grad_scaler is not None:
            raise NotImplementedError("FusedAdam.step(grad_scaler=...): unscale with torch.amp.GradScaler.unscale_ "
                                      "before the step, or pass the inverse scale through multi_tensor_adam")
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            if not group["params"]:
                continue
            step = self._step_value(group)
            lr = self._lr_value(group)
            b1, b2 = group["betas"]
            buckets = {}
            quantized = []
            for p in group["params"]:
                g = getattr(p, "decoupled_grad", None) if self.use_decoupled_grad else p.grad
                if g is None:
                    continue
                if getattr(p, "grad_added_to_main_grad", False) and g.numel() > 1 and g.stride() == (0,) * g.dim():
                    continue  # placeholder returned when the wgrad GEMM accumulated into main_grad
                g = _local(g)
                if not g.is_contiguous():
                    g = g.contiguous()
                key_param, p = p, _local(p)
                if p.numel() == 0:
                    continue    # this rank's shard of a small sharded parameter is empty
                st = self._init_state(key_param, p)
                if isinstance(p, QuantizedTensor):
                    quantized.append((p, g, st))
                    continue
                mode = 2 if "param_remainder" in st else (1 if "master_param" in st else 0)
                key = (g.dtype, p.dtype, mode)
                b = buckets.setdefault(key, [[], [], [], [], []])
                b[0].append(g)
                b[1].append(p.data)
                b[2].append(st["exp_avg"])
                b[3].append(st["exp_avg_sq"])
                if mode:
                    b[4].append(st["param_remainder"] if mode == 2 else st["master_param"])
            for (gd, pd, mode), lists in buckets.items():
                ls = lists if mode else lists[:4]
                ops.multi_tensor_adam(ls, lr, b1, b2, group["eps"], step, self.adam_w_mode,
                                      group["bias_correction"], group["weight_decay"], remainders=mode == 2)
            for p, g, st in quantized:
                # quantized (FP8 / block-scaled) parameters: update the fp32 master, then re-quantize in place
                tmp = torch.empty_like(st["master_param"])
                ops.multi_tensor_adam([[g.float()], [tmp], [st["exp_avg"]], [st["exp_avg_sq"]], [st["master_param"]]],
                                      lr, b1, b2, group["eps"], step, self.adam_w_mode,
                                      group["bias_correction"], group["weight_decay"])
                p.quantize_(st["master_param"])
        bump_weights_epoch()
        return loss

    def state_dict(self):  # type: ignore[override]
        sd = super().state_dict()
        for g in sd["param_groups"]:
            g.pop("_lr_dev", None)
            if isinstance(g.get("step"), torch.Tensor):
                g["step"] = int(g["step"].item())
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
