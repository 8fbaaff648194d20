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
        for name, dt in (("exp_avg_dtype", exp_avg_dtype), ("exp_avg_sq_dtype", exp_avg_sq_dtype)):
            if dt not in (torch.float32, torch.bfloat16, torch.float16, torch.uint8):
                raise RuntimeError(f"{name} must be float32, bfloat16, float16 or uint8 (FP8 E4M3), got {dt}")
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
        # fp32 / bf16 moments are read and written by the multi-tensor kernel itself (both must then share a dtype);
        # float16 and uint8 (FP8 E4M3 bytes) moments are stored divided by a per-tensor scale and pass through fp32
        # temporaries around the kernel: less memory, two more passes over the state
        self.name_to_dtype_map = {"exp_avg": exp_avg_dtype, "exp_avg_sq": exp_avg_sq_dtype,
                                  "master_param": master_weight_dtype}
        self._scaled_states = any(d in (torch.float16, torch.uint8) for d in (exp_avg_dtype, exp_avg_sq_dtype)) \
            or exp_avg_dtype != exp_avg_sq_dtype
        self.state_dtype = torch.float32 if self._scaled_states else exp_avg_dtype   # dtype the kernel sees
        self._scales = {}      # param -> {state name -> fp32 scale tensor [1]} for the scaled states
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
            for name in ("exp_avg", "exp_avg_sq"):
                dt = self.name_to_dtype_map[name] if self._scaled_states else self.state_dtype
                st[name] = torch.zeros(base.shape, dtype=dt, device=base.device)
                if dt in (torch.float16, torch.uint8):
                    self._scales.setdefault(key, {})[name] = torch.ones(1, dtype=torch.float32, device=base.device)
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

    # ---- optimizer states in high precision (reference: optimizers/fused_adam.py, get_unscaled_state /
    # set_scaled_state / initialize_state; distributed optimizers use them to save and re-shard the states)
    _FP8_MAX, _FP16_MAX = 448.0, 65504.0

    def _decode(self, key, name, stored):
        dt = stored.dtype
        if dt == torch.uint8:
            return stored.view(torch.float8_e4m3fn).float() * self._scales[key][name]
        if dt == torch.float16:
            return stored.float() * self._scales[key][name]
        return stored.float() if dt == torch.bfloat16 else stored

    def _encode(self, key, name, value, stored):
        dt = stored.dtype
        if dt in (torch.uint8, torch.float16):
            scale = self._scales[key][name]
            amax = value.abs().amax().float().clamp(min=1e-30)
            scale.copy_((amax / (self._FP8_MAX if dt == torch.uint8 else self._FP16_MAX)).reshape(1))
            q = value.float() / scale
            if dt == torch.uint8:
                stored.copy_(q.clamp(-self._FP8_MAX, self._FP8_MAX).to(torch.float8_e4m3fn).view(torch.uint8))
            else:
                stored.copy_(q.to(torch.float16))
        else:
            stored.copy_(value)

    def get_unscaled_state(self, param, state_name: str, skip_unscale: bool = False) -> torch.Tensor:
        """The state ``exp_avg`` / ``exp_avg_sq`` / ``master_param`` of ``param`` in fp32 (bf16 states come back as
        bf16 with ``skip_unscale``; a master weight kept as 16-bit remainders comes back as the int16 remainders).
        Sharded (``DTensor``) parameters give the local shard's state."""
        st = self.state[param]
        if state_name == "master_param" and "param_remainder" in st:
            return st["param_remainder"]
        stored = _local(st[state_name])
        if stored.dtype == torch.bfloat16 and skip_unscale:
            return stored
        return self._decode(param, state_name, stored)

    def set_scaled_state(self, param, state_name: str, unscaled_state: torch.Tensor) -> None:
        """Overwrite a state from its fp32 value (scaled and rounded to the state's storage dtype); the int16
        remainders for a master weight kept as remainders."""
        st = self.state[param]
        if state_name == "master_param" and self.store_param_remainders and _local(param).dtype == torch.bfloat16 \
                and not isinstance(_local(param), QuantizedTensor):
            assert unscaled_state.dtype == torch.int16, "a master weight kept as remainders is set from int16"
            st["param_remainder"] = unscaled_state.clone() if "param_remainder" not in st else \
                st["param_remainder"].copy_(unscaled_state)
            return
        assert unscaled_state.dtype == torch.float32, "states are set from fp32 values"
        if "exp_avg" not in st:
            self._init_state(param, _local(param))
        if state_name == "master_param" and "master_param" not in st:
            st["master_param"] = unscaled_state.clone()
            return
        self._encode(param, state_name, unscaled_state, _local(st[state_name]))

    def initialize_state(self, param, store_param_remainders: bool = False) -> None:
        """Create the states of ``param`` before the first step (moments zero, master weight from the parameter)."""
        if store_param_remainders and not self.store_param_remainders:
            raise RuntimeError("the optimizer was built without store_param_remainders")
        self._init_state(param, _local(param))

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
            rescale = []        # (param, state, fp32 exp_avg, fp32 exp_avg_sq) of scaled states, written back below
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
                    quantized.append((key_param, p, g, st))
                    continue
                mode = 2 if "param_remainder" in st else (1 if "master_param" in st else 0)
                key = (g.dtype, p.dtype, mode)
                b = buckets.setdefault(key, [[], [], [], [], []])
                b[0].append(g)
                b[1].append(p.data)
                if self._scaled_states:
                    m, v = (self._decode(key_param, n, st[n]).contiguous() for n in ("exp_avg", "exp_avg_sq"))
                    rescale.append((key_param, st, m, v))
                    b[2].append(m)
                    b[3].append(v)
                    if mode:
                        b[4].append(st["param_remainder"] if mode == 2 else st["master_param"])
                    continue
                b[2].append(st["exp_avg"])
                b[3].append(st["exp_avg_sq"])
                if mode:
                    b[4].append(st["param_remainder"] if mode == 2 else st["master_param"])
            for (gd, pd, mode), lists in buckets.items():
                ls = lists if mode else lists[:4]
                ops.multi_tensor_adam(ls, lr, b1, b2, group["eps"], step, self.adam_w_mode,
                                      group["bias_correction"], group["weight_decay"], remainders=mode == 2)
            for kp, p, g, st in quantized:
                # quantized (FP8 / block-scaled) parameters: update the fp32 master, then re-quantize in place
                tmp = torch.empty_like(st["master_param"])
                if self._scaled_states:
                    m, v = (self._decode(kp, n, st[n]).contiguous() for n in ("exp_avg", "exp_avg_sq"))
                    rescale.append((kp, st, m, v))
                else:
                    m, v = st["exp_avg"], st["exp_avg_sq"]
                ops.multi_tensor_adam([[g.float()], [tmp], [m], [v], [st["master_param"]]],
                                      lr, b1, b2, group["eps"], step, self.adam_w_mode,
                                      group["bias_correction"], group["weight_decay"])
                p.quantize_(st["master_param"])
            for kp, st, m, v in rescale:
                for name, val in (("exp_avg", m), ("exp_avg_sq", v)):
                    if val is not st[name]:
                        self._encode(kp, name, val, st[name])
        bump_weights_epoch()
        return loss

    def state_dict(self):  # type: ignore[override]
        sd = super().state_dict()
        for g in sd["param_groups"]:
            g.pop("_lr_dev", None)
            if isinstance(g.get("step"), torch.Tensor):
                g["step"] = int(g["step"].item())
        params = [p for g in self.param_groups for p in g["params"]]
        for idx, st in sd["state"].items():
            for k in ("exp_avg", "exp_avg_sq"):
                if k in st and st[k].dtype != torch.float32:
                    key = params[idx] if isinstance(idx, int) and idx < len(params) else None
                    # checkpoints always hold unscaled fp32 moments
                    st[k] = self._decode(key, k, st[k]) if st[k].dtype in (torch.uint8, torch.float16) else st[k].float()
        return sd

    def load_state_dict(self, state_dict):  # type: ignore[override]
        super().load_state_dict(state_dict)
        for key, st in self.state.items():
            for k in ("exp_avg", "exp_avg_sq"):
                if k not in st:
                    continue
                want = self.name_to_dtype_map[k] if self._scaled_states else self.state_dtype
                if want in (torch.uint8, torch.float16):
                    value = st[k].float()
                    st[k] = torch.zeros(value.shape, dtype=want, device=value.device)
                    self._scales.setdefault(key, {})[k] = torch.ones(1, dtype=torch.float32, device=value.device)
                    self._encode(key, k, value, st[k])
                elif st[k].dtype != want:
                    st[k] = st[k].to(want)
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
