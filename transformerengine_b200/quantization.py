"""``autocast`` and the global quantization state.

``with autocast(enabled=True, recipe=R, amax_reduction_group=G):`` makes every
module of this library run its GEMMs in the recipe's low-precision format.
For delayed scaling, amaxes recorded during the region are reduced (MAX over
``G``) and turned into the next step's scales when the outermost region exits
(reference: ``pytorch/quantization.py:645-843, 972-1064, 1067-1116``).
"""
from __future__ import annotations

import dataclasses

import os
from contextlib import contextmanager
from typing import Dict, List, Optional, Tuple

import torch

from .common.recipe import (CustomRecipe, DelayedScaling, Float8BlockScaling, Float8CurrentScaling, Format,
                            MXFP8BlockScaling, NVFP4BlockScaling, Recipe)
from .ops.ref import quant as Q
from .tensor import (Float8BlockQuantizer, Float8CurrentScalingQuantizer, Float8Quantizer, MXFP8Quantizer,
                     NVFP4Quantizer)


def _device_cc() -> Optional[Tuple[int, int]]:
    if torch.cuda.is_available():
        return torch.cuda.get_device_capability()
    return None


def is_fp8_available(return_reason: bool = False):
    """FP8 execution needs sm_89+; on CPU the quantize-dequantize reference path is used."""
    cc = _device_cc()
    ok = cc is None or cc >= (8, 9)
    reason = "" if ok else "Device compute capability 8.9 or higher required for FP8 execution."
    return (ok, reason) if return_reason else ok


def is_mxfp8_available(return_reason: bool = False):
    cc = _device_cc()
    ok = cc is None or cc >= (10, 0)
    reason = "" if ok else "Device compute capability 10.0 or higher required for MXFP8 execution."
    return (ok, reason) if return_reason else ok


def is_nvfp4_available(return_reason: bool = False):
    cc = _device_cc()
    ok = cc is None or cc >= (10, 0)
    reason = "" if ok else "Device compute capability 10.0 or higher required for NVFP4 execution."
    return (ok, reason) if return_reason else ok


def is_fp8_block_scaling_available(return_reason: bool = False):
    cc = _device_cc()
    ok = cc is None or cc >= (9, 0)
    reason = "" if ok else "Device compute capability 9.0 or higher required for FP8 block scaling."
    return (ok, reason) if return_reason else ok


check_fp8_support = lambda: is_fp8_available(True)  # noqa: E731
check_mxfp8_support = lambda: is_mxfp8_available(True)  # noqa: E731
check_nvfp4_support = lambda: is_nvfp4_available(True)  # noqa: E731
check_fp8_block_scaling_support = lambda: is_fp8_block_scaling_available(True)  # noqa: E731


def get_default_fp8_recipe() -> Recipe:
    """MXFP8 on Blackwell, delayed scaling elsewhere."""
    cc = _device_cc()
    if cc is not None and cc >= (10, 0):
        return MXFP8BlockScaling()
    return DelayedScaling()


get_default_recipe = get_default_fp8_recipe


def get_fp8_torch_dtype(recipe: Recipe, fprop_tensor: bool = True) -> torch.dtype:
    fmt = getattr(recipe, "fp8_format", Format.HYBRID)
    if fmt == Format.E4M3 or (fmt == Format.HYBRID and fprop_tensor):
        return torch.float8_e4m3fn
    return torch.float8_e5m2


def get_fp8_te_dtype(recipe: Recipe, fprop_tensor: bool = True):
    """The FP8 format of a recipe's forward / backward tensors as the library's ``DType`` enum."""
    from .constants import DType
    return DType.kFloat8E4M3 if get_fp8_torch_dtype(recipe, fprop_tensor) == torch.float8_e4m3fn else DType.kFloat8E5M2


def get_fp4_te_dtype(recipe: Recipe):
    from .constants import DType
    return DType.kFloat4E2M1


def get_fp8_max(recipe: Recipe, fprop_tensor: bool = True) -> float:
    fmt = getattr(recipe, "fp8_format", Format.HYBRID)
    return fmt.value.max_fwd if fprop_tensor else fmt.value.max_bwd


def check_recipe_support(recipe: Recipe) -> None:
    if isinstance(recipe, MXFP8BlockScaling):
        ok, why = is_mxfp8_available(True)
    elif isinstance(recipe, NVFP4BlockScaling):
        ok, why = is_nvfp4_available(True)
    elif isinstance(recipe, Float8BlockScaling):
        ok, why = is_fp8_block_scaling_available(True)
    else:
        ok, why = is_fp8_available(True)
    assert ok, why


# --------------------------------------------------------------------------- recipe state

@dataclasses.dataclass(frozen=True)
class QuantizerRole:
    """Which tensor slot asks a ``CustomRecipe`` factory for a quantizer: the kind of module (``"linear"``,
    ``"grouped_linear"``, ``"dpa"``), the tensor (``"input"``, ``"weight"``, ``"output"``, ``"grad_output"``,
    ``"grad_input"``) and the module instance's name.  Factories may also be handed the plain strings this
    library uses (``"linear_input"`` ...); ``custom_recipes.quantizer_factories.tensor_type`` reads both.
    (Reference: ``pytorch/quantization.py:57``.)"""

    module_type: str = ""
    tensor_type: str = ""
    name: str = ""

    def __str__(self) -> str:
        parts = [f"{k}={v}" for k, v in (("module_type", self.module_type), ("tensor_type", self.tensor_type),
                                         ("name", self.name)) if v]
        return "|".join(parts) if parts else "QuantizerRole()"


@dataclasses.dataclass(frozen=True)
class QuantizerRequest:
    """Base class of the requests a ``CustomRecipe`` factory may return instead of a quantizer when the quantizer
    needs state that the library manages.  A request may also stand in for a child of a ``HybridQuantizer``."""

    _is_quantizer_request = True


@dataclasses.dataclass(frozen=True)
class DelayedScalingRequest(QuantizerRequest):
    """Ask for a per-tensor FP8 quantizer whose scale follows an amax history kept by the library."""

    fp8_format: object = None          # recipe.Format; None = HYBRID
    margin: int = 0
    amax_history_len: int = 1024
    amax_compute_algo: object = "max"
    scaling_factor_compute_algo: object = None
    reduce_amax: bool = True


class RecipeState:
    """Per-module, per-direction quantization state; builds the quantizers.

    ``mode`` is ``"forward"`` (slots: input, weight, output per GEMM) or
    ``"backward"`` (slots: grad_output, grad_input per GEMM).
    """

    @staticmethod
    def create(recipe: Recipe, *, mode: str, num_quantizers: int = 1, device=None) -> "RecipeState":
        cls = None
        if recipe.delayed():
            cls = DelayedScalingRecipeState
        elif recipe.mxfp8():
            cls = MXFP8BlockScalingRecipeState
        elif recipe.float8_current_scaling():
            cls = Float8CurrentScalingRecipeState
        elif recipe.float8_block_scaling():
            cls = Float8BlockScalingRecipeState
        elif recipe.nvfp4():
            cls = NVFP4BlockScalingRecipeState
        elif recipe.custom():
            cls = CustomRecipeState
        else:
            raise ValueError(f"{recipe.__class__.__name__} is not supported")
        return cls(recipe, mode=mode, num_quantizers=num_quantizers, device=device)

    def __init__(self, recipe, *, mode, num_quantizers, device):
        self.recipe, self.mode, self.num_quantizers = recipe, mode, num_quantizers
        self.device = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
        self.dtype = get_fp8_torch_dtype(recipe, fprop_tensor=(mode == "forward"))

    def make_quantizers(self) -> list:
        raise NotImplementedError


class DelayedScalingRecipeState(RecipeState):
    def __init__(self, recipe, *, mode, num_quantizers, device):
        super().__init__(recipe, mode=mode, num_quantizers=num_quantizers, device=device)
        self.scale = torch.ones(num_quantizers, dtype=torch.float32, device=self.device)
        self.amax_history = torch.zeros(recipe.amax_history_len, num_quantizers, dtype=torch.float32,
                                        device=self.device)

    def make_quantizers(self):
        return [Float8Quantizer(self.scale[i], self.amax_history[0][i].reshape(1), self.dtype)
                for i in range(self.num_quantizers)]


class Float8CurrentScalingRecipeState(RecipeState):
    def make_quantizers(self):
        r = self.recipe
        out = []
        for i in range(self.num_quantizers):
            if self.mode == "forward":
                qp = r.fp8_quant_fwd_weight if i % 3 == 1 else r.fp8_quant_fwd_inp
            else:
                qp = r.fp8_quant_bwd_grad
            out.append(Float8CurrentScalingQuantizer(
                self.dtype, device=self.device, force_pow_2_scales=qp.power_2_scale or r.use_power_2_scales,
                amax_epsilon=qp.amax_epsilon))
        return out


class MXFP8BlockScalingRecipeState(RecipeState):
    def make_quantizers(self):
        # enable_2d_quantization: weights (slot 1 of every forward GEMM) use 32 x 32 blocks, so that their row-wise
        # and column-wise copies hold the same values
        two_d = self.mode == "forward" and getattr(self.recipe, "enable_2d_quantization", False)
        return [MXFP8Quantizer(self.dtype, with_2d_quantization=two_d and i % 3 == 1)
                for i in range(self.num_quantizers)]


class Float8BlockScalingRecipeState(RecipeState):
    def make_quantizers(self):
        r = self.recipe
        out = []
        for i in range(self.num_quantizers):
            if self.mode == "forward":
                is_w = i % 3 == 1
                qp = r.fp8_quant_fwd_weight if is_w else r.fp8_quant_fwd_inp
                dim = r.w_block_scaling_dim if is_w else r.x_block_scaling_dim
            else:
                qp, dim = r.fp8_quant_bwd_grad, r.grad_block_scaling_dim
            out.append(Float8BlockQuantizer(self.dtype, amax_epsilon=qp.amax_epsilon,
                                            force_pow_2_scales=qp.power_2_scale, block_scaling_dim=dim))
        return out


class NVFP4BlockScalingRecipeState(RecipeState):
    def make_quantizers(self):
        r = self.recipe
        out = []
        for i in range(self.num_quantizers):
            if self.mode == "forward":
                qp = r.fp4_quant_fwd_weight if i % 3 == 1 else r.fp4_quant_fwd_inp
            else:
                qp = r.fp4_quant_bwd_grad
            # adaptive (4-over-6) block scaling of the forward tensors the recipe names; gradients keep the
            # standard scaling (reference: quantization.py, NVFP4BlockScalingRecipeState.make_quantizers)
            is_weight = self.mode == "forward" and i % 3 == 1
            scope = "weights" if is_weight else "activations"
            adaptive = self.mode == "forward" and r.nvfp4_4over6 in ("all", scope)
            if adaptive and (qp.random_hadamard_transform or qp.stochastic_rounding):
                raise ValueError("NVFP4 4over6 quantization does not support the random Hadamard transform or "
                                 "stochastic rounding: set disable_rht=True (and disable_stochastic_rounding=True)")
            bound = 256 if adaptive and r.nvfp4_4over6_e4m3_use_256 in ("all", scope) else 448
            out.append(NVFP4Quantizer(with_rht=qp.random_hadamard_transform,
                                      with_2d_quantization=qp.fp4_2d_quantization,
                                      stochastic_rounding=qp.stochastic_rounding,
                                      row_scaled_nvfp4=(self.mode == "forward" and not is_weight
                                                        and r.row_scaled_activation),
                                      nvfp4_use_4over6=adaptive, nvfp4_e4m3_max=bound,
                                      nvfp4_4over6_err_mode=r.nvfp4_4over6_err_mode))
        return out


class CustomRecipeState(RecipeState):
    _FWD = ("linear_input", "linear_weight", "linear_output")
    _BWD = ("linear_grad_output", "linear_grad_input")

    delayed: Optional["DelayedScalingRecipeState"] = None   # state behind the slots that asked for delayed scaling

    def make_quantizers(self):
        roles = self._FWD if self.mode == "forward" else self._BWD
        from .tensor.hybrid import HybridQuantizer

        out = [self.recipe.qfactory(roles[i % len(roles)]) for i in range(self.num_quantizers)]
        # (place to put the quantizer, request): whole slots, and children of hybrid quantizers
        asked = []
        for i, q in enumerate(out):
            if isinstance(q, DelayedScalingRequest):
                asked.append(((out, i), q))
            elif isinstance(q, HybridQuantizer):
                for side in ("rowwise_quantizer", "columnwise_quantizer"):
                    if isinstance(getattr(q, side), DelayedScalingRequest):
                        asked.append(((q, side), getattr(q, side)))
        if asked:
            first = asked[0][1]
            if any(r != first for _, r in asked):
                raise ValueError("all DelayedScalingRequest objects of one module must carry the same parameters")
            kw = dict(margin=first.margin, amax_history_len=first.amax_history_len,
                      amax_compute_algo=first.amax_compute_algo,
                      scaling_factor_compute_algo=first.scaling_factor_compute_algo, reduce_amax=first.reduce_amax)
            if first.fp8_format is not None:
                kw["fp8_format"] = first.fp8_format
            self.delayed = DelayedScalingRecipeState(DelayedScaling(**kw), mode=self.mode, num_quantizers=len(asked),
                                                     device=self.device)
            for q, ((holder, where), _) in zip(self.delayed.make_quantizers(), asked):
                if isinstance(holder, list):
                    holder[where] = q
                else:
                    holder.set_child(where, q)
        return out


# --------------------------------------------------------------------------- delayed-scaling update
def _default_get_amax(history: torch.Tensor, algo) -> torch.Tensor:
    if callable(algo):
        return algo(history)
    return history.amax(dim=0) if algo == "max" else history[0].clone()


def _roll_and_zero_out(history: torch.Tensor) -> None:
    if history.shape[0] > 1:
        history.copy_(torch.roll(history, -1, 0))
    history[0].zero_()


def update_delayed_scaling_state(state: DelayedScalingRecipeState, reduced_amax: Optional[torch.Tensor] = None):
    """New scales from the amax history, then roll the history (slot 0 is cleared)."""
    r = state.recipe
    if reduced_amax is not None:
        state.amax_history[0].copy_(reduced_amax)
    fmax = get_fp8_max(r, fprop_tensor=(state.mode == "forward"))
    from .ops import _ext

    if (_ext.use_cuda(state.amax_history) and hasattr(_ext.get(), "delayed_scaling_update")
            and not callable(r.scaling_factor_compute_algo) and r.amax_compute_algo in ("max", "most_recent")
            and state.amax_history.is_contiguous() and state.scale.is_contiguous()):
        # one launch: history max, new scales, roll + clear (csrc/quant/recipe_kernels.cu)
        _ext.get().delayed_scaling_update(state.amax_history, state.scale, float(fmax), int(r.margin),
                                          r.amax_compute_algo == "most_recent")
        return
    amax = _default_get_amax(state.amax_history, r.amax_compute_algo)
    if callable(r.scaling_factor_compute_algo):
        new_scale = r.scaling_factor_compute_algo(amax, state.scale, fmax, r)
    else:
        new_scale = Q.compute_scale_from_amax(amax, fmax, r.margin, False, 0.0, prev_scale=state.scale)
    state.scale.copy_(new_scale)
    _roll_and_zero_out(state.amax_history)


# --------------------------------------------------------------------------- global state
class FP8GlobalStateManager:
    """Process-wide quantization state shared by all modules."""

    FP8_ENABLED = False
    FP8_CALIBRATION = False
    FP8_RECIPE: Optional[Recipe] = None
    FP8_DISTRIBUTED_GROUP = None
    FP8_PARAMETERS = False
    HIGH_PRECISION_INIT_VAL = False
    FP8_MODEL_INIT_RECIPE: Optional[Recipe] = None
    IS_FIRST_FP8_MODULE = False
    FP8_GRAPH_CAPTURING = False
    FP8_AUTOCAST_DEPTH = 0
    # delayed-scaling states that recorded amaxes in the current region, per direction
    _pending: Dict[str, List[DelayedScalingRecipeState]] = {"forward": [], "backward": []}
    _groups: Dict[int, object] = {}
    skip_fp8_weight_update_tensor: Optional[torch.Tensor] = None

    @classmethod
    def reset(cls) -> None:
        cls.FP8_ENABLED = False
        cls.FP8_CALIBRATION = False
        cls.FP8_RECIPE = None
        cls.FP8_DISTRIBUTED_GROUP = None
        cls.FP8_PARAMETERS = False
        cls.HIGH_PRECISION_INIT_VAL = False
        cls.FP8_MODEL_INIT_RECIPE = None
        cls.IS_FIRST_FP8_MODULE = False
        cls.FP8_GRAPH_CAPTURING = False
        cls.FP8_AUTOCAST_DEPTH = 0
        cls._pending = {"forward": [], "backward": []}
        cls._groups = {}
        cls.skip_fp8_weight_update_tensor = None

    @classmethod
    def is_fp8_enabled(cls) -> bool:
        return cls.FP8_ENABLED

    @classmethod
    def is_fp8_calibration(cls) -> bool:
        return cls.FP8_CALIBRATION

    @classmethod
    def with_fp8_parameters(cls) -> bool:
        return cls.FP8_PARAMETERS

    @classmethod
    def with_high_precision_init_val(cls) -> bool:
        return cls.HIGH_PRECISION_INIT_VAL

    @classmethod
    def fp8_graph_capturing(cls) -> bool:
        return cls.FP8_GRAPH_CAPTURING

    @classmethod
    def is_first_fp8_module(cls) -> bool:
        """True for the first module that runs in the current forward; that module's
        backward (the last one to run) triggers the backward amax reduction."""
        tmp = cls.IS_FIRST_FP8_MODULE
        cls.IS_FIRST_FP8_MODULE = False
        return tmp

    @classmethod
    def get_fp8_recipe(cls) -> Recipe:
        return cls.FP8_RECIPE if cls.FP8_RECIPE is not None else get_default_fp8_recipe()

    @classmethod
    def get_fp8_group(cls):
        return cls.FP8_DISTRIBUTED_GROUP

    @classmethod
    def get_autocast_state(cls):
        return (cls.FP8_ENABLED, cls.FP8_CALIBRATION, cls.FP8_RECIPE, cls.FP8_DISTRIBUTED_GROUP,
                cls.IS_FIRST_FP8_MODULE, cls.FP8_GRAPH_CAPTURING)

    @classmethod
    def set_autocast_state(cls, st) -> None:
        (cls.FP8_ENABLED, cls.FP8_CALIBRATION, cls.FP8_RECIPE, cls.FP8_DISTRIBUTED_GROUP,
         cls.IS_FIRST_FP8_MODULE, cls.FP8_GRAPH_CAPTURING) = st

    get_fp8_autocast_state = get_autocast_state
    set_fp8_autocast_state = set_autocast_state

    @classmethod
    def add_pending(cls, state: RecipeState, forward: bool = True) -> None:
        """A delayed-scaling state recorded amaxes: reduce and update it at region exit."""
        if isinstance(state, DelayedScalingRecipeState):
            lst = cls._pending["forward" if forward else "backward"]
            if not any(s is state for s in lst):
                lst.append(state)
                cls._groups[id(state)] = cls.FP8_DISTRIBUTED_GROUP

    @classmethod
    def reduce_and_update_fp8_tensors(cls, forward: bool = True) -> None:
        """One all-reduce(MAX) over the concatenated amaxes, then per-state scale update."""
        key = "forward" if forward else "backward"
        states, cls._pending[key] = cls._pending[key], []
        if not states:
            return
        by_group: Dict[int, list] = {}
        for s in states:
            g = cls._groups.pop(id(s), None)
            by_group.setdefault(id(g), [g, []])[1].append(s)
        for g, lst in by_group.values():
            reduce = [s for s in lst if s.recipe.reduce_amax]
            if reduce and g is not None and torch.distributed.is_initialized() \
                    and torch.distributed.get_world_size(g) > 1:
                flat = torch.cat([s.amax_history[0] for s in reduce])
                torch.distributed.all_reduce(flat, op=torch.distributed.ReduceOp.MAX, group=g)
                off = 0
                for s in reduce:
                    n = s.amax_history.shape[1]
                    s.amax_history[0].copy_(flat[off:off + n])
                    off += n
            for s in lst:
                update_delayed_scaling_state(s)

    @classmethod
    def autocast_enter(cls, enabled, calibrating, recipe, group, _graph=False) -> None:
        recipe = recipe if recipe is not None else get_default_fp8_recipe()
        cls.FP8_ENABLED = enabled
        cls.FP8_CALIBRATION = calibrating
        cls.FP8_RECIPE = recipe
        cls.FP8_DISTRIBUTED_GROUP = group
        cls.FP8_GRAPH_CAPTURING = _graph
        if cls.FP8_AUTOCAST_DEPTH == 0:
            cls.IS_FIRST_FP8_MODULE = True
        cls.FP8_AUTOCAST_DEPTH += 1
        if enabled:
            check_recipe_support(recipe)

    @classmethod
    def autocast_exit(cls, enabled, _graph=False) -> None:
        cls.FP8_AUTOCAST_DEPTH -= 1
        if enabled and cls.FP8_AUTOCAST_DEPTH == 0 and not _graph and torch.is_grad_enabled():
            cls.reduce_and_update_fp8_tensors(forward=True)


@contextmanager
def autocast(enabled: bool = True, calibrating: bool = False, recipe: Optional[Recipe] = None,
             amax_reduction_group=None, _graph: bool = False):
    """Run the enclosed modules with quantized GEMMs according to ``recipe``."""
    saved = FP8GlobalStateManager.get_autocast_state()
    FP8GlobalStateManager.autocast_enter(enabled, calibrating, recipe, amax_reduction_group, _graph)
    try:
        yield
    finally:
        FP8GlobalStateManager.set_autocast_state(saved)
        FP8GlobalStateManager.autocast_exit(enabled, _graph)


@contextmanager
def fp8_autocast(enabled: bool = True, calibrating: bool = False, fp8_recipe: Optional[Recipe] = None,
                 fp8_group=None, _graph: bool = False):
    """Older spelling of :func:`autocast`."""
    with autocast(enabled=enabled, calibrating=calibrating, recipe=fp8_recipe, amax_reduction_group=fp8_group,
                  _graph=_graph):
        yield


@contextmanager
def quantized_model_init(enabled: bool = True, recipe: Optional[Recipe] = None,
                         preserve_high_precision_init_val: bool = False):
    """Create module parameters directly as quantized tensors (no 16-bit copy kept)."""
    st = (FP8GlobalStateManager.FP8_PARAMETERS, FP8GlobalStateManager.FP8_MODEL_INIT_RECIPE,
          FP8GlobalStateManager.HIGH_PRECISION_INIT_VAL)
    FP8GlobalStateManager.FP8_PARAMETERS = enabled
    FP8GlobalStateManager.FP8_MODEL_INIT_RECIPE = recipe if recipe is not None else get_default_fp8_recipe()
    FP8GlobalStateManager.HIGH_PRECISION_INIT_VAL = preserve_high_precision_init_val
    try:
        yield
    finally:
        (FP8GlobalStateManager.FP8_PARAMETERS, FP8GlobalStateManager.FP8_MODEL_INIT_RECIPE,
         FP8GlobalStateManager.HIGH_PRECISION_INIT_VAL) = st


fp8_model_init = quantized_model_init


def get_align_size_for_quantization(recipe: Recipe) -> int:
    """Row alignment that expert slabs need for grouped quantized GEMMs."""
    if recipe.mxfp8():
        return 128  # one 128-row scale tile per slab boundary (tcgen05 scale layout)
    if recipe.nvfp4():
        return 128
    return 16
