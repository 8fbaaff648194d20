"""``Sequential`` container that fuses runs of basic operations (reference:
``pytorch/ops/sequential.py``, ``pytorch/ops/fuser.py:53,400``)."""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch

from . import ops as O
from .fused import ForkNorm, GroupedMLP, LinearChain
from ..modules.layernorm_linear import LayerNormLinear
from ..modules.layernorm_mlp import LayerNormMLP


class _Fused(torch.nn.Module):
    """A fused implementation standing in for ``span`` consecutive basic operations."""

    is_fused_op = True

    def __init__(self, impl: Callable, span: int, extra_inputs: int = 0, name: str = ""):
        super().__init__()
        self._impl = [impl]  # in a list: the fused module's parameters belong to the basic operations
        self.span, self.num_extra_inputs, self.num_extra_outputs, self.fusion = span, extra_inputs, 0, name

    def forward(self, x, *extra):
        return self._impl[0](x, *extra)


def _norm_kind(op) -> Optional[str]:
    if isinstance(op, O.LayerNorm):
        return "LayerNorm"
    if isinstance(op, O.RMSNorm):
        return "RMSNorm"
    return None


def _is_linear(op) -> bool:
    return isinstance(op, (O.BasicLinear, O.Linear)) and getattr(op, "parallel_mode", None) is None


def _share(dst: torch.nn.Module, name: str, p):
    if p is None:
        dst.register_parameter(name, None) if name in dst._parameters else setattr(dst, name, None)
    else:
        dst._parameters[name] = p


def _fuse_norm_linear(norm, lin) -> Callable:
    has_bias = getattr(lin, "bias", None) is not None
    m = LayerNormLinear(lin.in_features, lin.out_features, eps=norm.eps, bias=has_bias,
                        normalization=_norm_kind(norm), params_dtype=lin.weight.dtype, device="meta",
                        zero_centered_gamma=norm.zero_centered_gamma)
    _share(m, "layer_norm_weight", norm.weight)
    _share(m, "layer_norm_bias", getattr(norm, "bias", None))
    _share(m, "weight", lin.weight)
    if has_bias:
        _share(m, "bias", lin.bias)
    return m


def _fuse_norm_mlp(norm, fc1, act, fc2) -> Callable:
    has_bias = getattr(fc1, "bias", None) is not None
    ffn = fc2.in_features
    m = LayerNormMLP(fc1.in_features, ffn, eps=norm.eps, bias=has_bias, normalization=_norm_kind(norm),
                     activation=act.act_name, params_dtype=fc1.weight.dtype, device="meta",
                     zero_centered_gamma=norm.zero_centered_gamma)
    _share(m, "layer_norm_weight", norm.weight)
    _share(m, "layer_norm_bias", getattr(norm, "bias", None))
    _share(m, "fc1_weight", fc1.weight)
    _share(m, "fc2_weight", fc2.weight)
    if has_bias:
        _share(m, "fc1_bias", fc1.bias)
        _share(m, "fc2_bias", fc2.bias)
    return m


# user fusion passes: functions ``ops -> ops`` (reference: ``pytorch/ops/fuser.py`` register_*_fusion)
_FUSIONS_FIRST: List[Callable] = []
_FUSIONS_LAST: List[Callable] = []


def register_forward_backward_fusion(op_fusion_func: Callable, prepend: bool = False) -> None:
    """Register a fusion pass of your own: ``op_fusion_func(ops, *, recipe) -> updated ops`` receives the list of
    operations of a ``Sequential`` and may replace runs of them by a module that does their work (``recipe`` is the
    active quantization recipe or None).  A replacement is any ``torch.nn.Module`` called as
    ``module(x, *extra_inputs)``; it declares ``num_extra_inputs`` / ``num_extra_outputs`` when it consumes or
    produces extra tensors, and its backward is whatever autograd records for it.  ``prepend=True`` runs the pass
    before the built-in fusions (so it sees the basic operations), the default after them."""
    (_FUSIONS_FIRST if prepend else _FUSIONS_LAST).append(op_fusion_func)


def register_forward_fusion(op_fusion_func: Callable, prepend: bool = False) -> None:
    """Same registry as ``register_forward_backward_fusion``: a fused module here always carries both passes (its
    backward is its autograd graph), so there is no separate forward-only pass."""
    register_forward_backward_fusion(op_fusion_func, prepend)


def register_backward_fusion(op_fusion_func: Callable, prepend: bool = False) -> None:
    raise NotImplementedError("backward passes are not fused separately here: a fused module owns its backward "
                              "through autograd; register the pair with register_forward_backward_fusion")


def unregister_fusion(op_fusion_func: Callable) -> None:
    for lst in (_FUSIONS_FIRST, _FUSIONS_LAST):
        while op_fusion_func in lst:
            lst.remove(op_fusion_func)


def _active_recipe():
    from ..quantization import FP8GlobalStateManager
    return FP8GlobalStateManager.get_fp8_recipe() if FP8GlobalStateManager.is_fp8_enabled() else None


def _backward_override():
    return getattr(_active_recipe(), "backward_override", None)


def fuse_operations(ops: List[torch.nn.Module]) -> List[torch.nn.Module]:
    """Greedy longest-match fusion of a list of basic operations (user passes before and after the built-in one)."""
    ops = list(ops)
    for fn in _FUSIONS_FIRST:
        ops = list(fn(ops, recipe=_active_recipe()))
    if not _backward_override():
        # the fused operations bring their own quantized backward passes; under recipe.backward_override the basic
        # operations run instead (their modules implement the 16-bit backward)
        ops = _builtin_fusions(ops)
    for fn in _FUSIONS_LAST:
        ops = list(fn(ops, recipe=_active_recipe()))
    return ops


def _plain_act(op) -> bool:
    """An activation the fused modules can absorb (an interleaved gated layout runs as a basic operation)."""
    return isinstance(op, O._Activation) and op.glu_interleave_size is None


def _builtin_fusions(ops: List[torch.nn.Module]) -> List[torch.nn.Module]:
    out: List[torch.nn.Module] = []
    i = 0
    while i < len(ops):
        w = ops[i:i + 4]
        if (len(w) == 4 and _norm_kind(w[0]) and _is_linear(w[1]) and _plain_act(w[2])
                and _is_linear(w[3]) and (getattr(w[1], "bias", None) is None) == (getattr(w[3], "bias", None) is None)
                and w[1].out_features == w[3].in_features * (2 if w[2].act_name in ("swiglu", "geglu", "reglu") else 1)):
            out.append(_Fused(_fuse_norm_mlp(*w), 4, name="norm_mlp"))
            i += 4
            continue
        if (len(w) >= 3 and isinstance(w[0], O.GroupedLinear) and isinstance(w[1], O.ScaledSwiGLU)
                and w[1].glu_interleave_size is None    # the fused expert MLP reads [gates | linear units]
                and isinstance(w[2], O.GroupedLinear) and w[0].num_groups == w[2].num_groups
                and w[0].out_features == 2 * w[2].in_features):
            out.append(GroupedMLP(w[0], w[1], w[2]))
            i += 3
            continue
        if len(w) >= 2 and _norm_kind(w[0]) and _is_linear(w[1]):
            out.append(_Fused(_fuse_norm_linear(w[0], w[1]), 2, name="norm_linear"))
            i += 2
            continue
        if len(w) >= 2 and isinstance(w[0], O.MakeExtraOutput) and _norm_kind(w[1]):
            # residual fork followed by a norm: the norm backward adds the fork's gradient itself
            out.append(ForkNorm(w[1], _norm_kind(w[1]) == "LayerNorm"))
            i += 2
            continue
        if _is_linear(ops[i]) and not getattr(ops[i], "return_bias", False):
            # Linear (+Bias) (+ConstantScale, bias-free only) (+Activation) (+AddExtraInput): one chain with a
            # fused backward (activation gradient + bias gradient + quantization in one kernel)
            lin, j = ops[i], i + 1
            own_bias = getattr(lin, "bias", None) is not None and getattr(lin, "apply_bias", True)
            bias_op, scale, act, add = None, 1.0, None, False
            if j < len(ops) and isinstance(ops[j], O.Bias) and not own_bias:
                bias_op, j = ops[j], j + 1
            if j < len(ops) and isinstance(ops[j], O.ConstantScale) and bias_op is None and not own_bias:
                scale, j = float(ops[j].scale), j + 1
            if j < len(ops) and _plain_act(ops[j]) and scale == 1.0:
                act, j = ops[j].act_name, j + 1
            if j < len(ops) and isinstance(ops[j], O.AddExtraInput):
                add, j = True, j + 1
            if j > i + 1:
                out.append(LinearChain(lin, bias_op, scale, act, add))
                i = j
                continue
        out.append(ops[i])
        i += 1
    return out


class Sequential(torch.nn.Module):
    """Runs its operations in order, fusing neighbours where this library has a fused kernel.

    ``forward(x, *extra_inputs)``: operations that declare ``num_extra_inputs`` take their
    additional tensors from ``extra_inputs`` in order; operations with ``num_extra_outputs``
    append to the returned tuple.
    """

    def __init__(self, *ops: torch.nn.Module):
        super().__init__()
        for i, op in enumerate(ops):
            self.add_module(str(i), op)
        self._plan: Optional[List[torch.nn.Module]] = None
        self._plan_key: Optional[Tuple[int, ...]] = None

    def __len__(self):
        return len(self._modules)

    def __getitem__(self, i):
        return list(self._modules.values())[i]

    def append(self, op: torch.nn.Module) -> "Sequential":
        self.add_module(str(len(self._modules)), op)
        self._plan = None
        return self

    def _get_plan(self) -> List[torch.nn.Module]:
        mods = list(self._modules.values())
        key = tuple(id(m) for m in mods)
        key = key + (len(_FUSIONS_FIRST), len(_FUSIONS_LAST), _backward_override())
        if self._plan is None or key != self._plan_key:
            self._plan, self._plan_key = fuse_operations(mods), key
        return self._plan

    def forward(self, x, *extra_inputs):
        extra = list(extra_inputs)
        outs = []
        for op in self._get_plan():
            n_in = getattr(op, "num_extra_inputs", 0)
            args, extra = extra[:n_in], extra[n_in:]
            y = op(x, *args)
            if getattr(op, "num_extra_outputs", 0):
                x, rest = y[0], y[1:]
                outs.extend(rest)
            else:
                x = y
        assert not extra, "more extra inputs than the operations consume"
        return (x, *outs) if outs else x
