"""Base class of all modules that run quantized GEMMs.

Holds the per-module recipe state (quantizers for input / weight / output of
each GEMM in the forward and grad_output / grad_input in the backward), the
quantized-weight cache, tensor-parallel settings and the ``_extra_state``
checkpoint entry (reference: ``pytorch/module/base.py:575-1480``).
"""
from __future__ import annotations

import io
import pickle
import warnings
from typing import Any, Dict, List, Optional

import torch

from ..common.recipe import DelayedScaling, Recipe
from ..quantization import FP8GlobalStateManager, RecipeState, DelayedScalingRecipeState
from ..tensor.base import QuantizedTensor, QuantizedTensorStorage, Quantizer

# bumped by the optimizers of this library after they update parameters in place
# through raw pointers (which does not touch torch's version counters)
_WEIGHTS_EPOCH = [0]


def bump_weights_epoch() -> None:
    _WEIGHTS_EPOCH[0] += 1


def weights_epoch() -> int:
    return _WEIGHTS_EPOCH[0]


# While set, quantized-weight caches are served without looking at parameter versions: a CUDA graph
# captured with cached weights re-quantizes them in place through ``requantize_cached_weights``.
_FREEZE_WEIGHT_CACHE = [False]


def freeze_weight_caches(flag: bool) -> bool:
    old = _FREEZE_WEIGHT_CACHE[0]
    _FREEZE_WEIGHT_CACHE[0] = bool(flag)
    return old


def get_distributed_world_size(group=None) -> int:
    if not torch.distributed.is_available() or not torch.distributed.is_initialized():
        return 1
    return torch.distributed.get_world_size(group=group)


def get_distributed_rank(group=None) -> int:
    if not torch.distributed.is_available() or not torch.distributed.is_initialized():
        return 0
    return torch.distributed.get_rank(group=group)


def _default_init(std: float = 0.023):
    def init_(t):
        return torch.nn.init.normal_(t, mean=0.0, std=std)
    return init_


def get_default_init_method():
    return _default_init(0.023)


_UNSAFE_PICKLE_ENV = "NVTE_ALLOW_UNSAFE_PICKLE_EXTRA_STATE"


class _SafeUnpickler(pickle.Unpickler):
    """Restricted unpickler for ``_extra_state``: recipe classes, tensors as torch rebuilds
    them, and inert builtin containers.  Anything callable beyond that is refused."""

    _BUILTINS = {"dict", "list", "tuple", "set", "frozenset", "int", "float", "bool", "str", "bytes", "complex",
                 "slice", "bytearray"}
    _TORCH = {("torch._utils", "_rebuild_tensor_v2"), ("torch._utils", "_rebuild_tensor"),
              ("torch", "Size"), ("torch", "device"), ("torch", "dtype"),
              ("torch.serialization", "_get_layout"), ("torch._tensor", "_rebuild_from_type_v2"),
              ("collections", "OrderedDict"),
              ("_codecs", "encode"), ("numpy.core.multiarray", "_reconstruct"), ("numpy", "ndarray"),
              ("numpy", "dtype"), ("numpy.core.multiarray", "scalar"), ("numpy._core.multiarray", "scalar"),
              ("numpy._core.multiarray", "_reconstruct")}

    # the only names of the recipe module a checkpoint may reference (classes and enums, no functions)
    _RECIPE_NAMES = {"Recipe", "DelayedScaling", "Float8CurrentScaling", "MXFP8BlockScaling", "Float8BlockScaling",
                     "NVFP4BlockScaling", "CustomRecipe", "Format", "_FormatHelper", "MMParams", "QParams"}

    @staticmethod
    def _storage_from_bytes(b):
        """Stand-in for ``torch.storage._load_from_bytes`` (which unpickles without restriction):
        the nested archive is read with the weights-only loader, which refuses arbitrary globals."""
        return torch.load(io.BytesIO(b), weights_only=True)

    def find_class(self, module, name):
        if module in ("transformer_engine.common.recipe", "transformerengine_b200.common.recipe"):
            if name not in self._RECIPE_NAMES:
                raise pickle.UnpicklingError(f"refusing to load {module}.{name} from _extra_state")
            from ..common import recipe as r
            return getattr(r, name)
        if (module, name) == ("torch.storage", "_load_from_bytes"):
            return self._storage_from_bytes
        if module == "builtins" and name in self._BUILTINS:
            return super().find_class(module, name)
        if (module, name) in self._TORCH:
            return super().find_class(module, name)
        if module == "torch" and (name.endswith("Storage") or name.endswith("Tensor")):
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"refusing to load {module}.{name} from _extra_state")


class TransformerEngineBaseModule(torch.nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.fp8 = False
        self.fp8_calibration = False
        self.fp8_initialized = False
        self.fp8_meta: Dict[str, Any] = {"recipe": None, "num_gemms": 1, "fp8_checkpoint": False}
        self.quantizers: Dict[str, List[Optional[Quantizer]]] = {"scaling_fwd": [], "scaling_bwd": []}
        self._states: Dict[str, Optional[RecipeState]] = {"scaling_fwd": None, "scaling_bwd": None}
        self._weight_cache: Dict[str, Any] = {}
        self._recompute_scales: List[torch.Tensor] = []  # forward scales of checkpointed runs awaiting recompute
        self.tp_group = None
        self.tp_size = 1
        self.sequence_parallel = False
        self.primary_weights_in_fp8 = FP8GlobalStateManager.with_fp8_parameters()
        self.preserve_high_precision_init_val = FP8GlobalStateManager.with_high_precision_init_val()
        self.name = None
        self.wgrad_store = None
        self.fuse_wgrad_accumulation = False

    # ------------------------------------------------------------------ TP
    def set_tensor_parallel_group(self, tp_group) -> None:
        self.tp_group = tp_group
        self.tp_size = get_distributed_world_size(tp_group)

    # ------------------------------------------------------------------ recipe state
    def init_fp8_metadata(self, num_gemms: int = 1) -> None:
        """(Re)build quantizers when entering a quantized region or when the recipe changed."""
        self.fp8 = FP8GlobalStateManager.is_fp8_enabled()
        self.fp8_calibration = FP8GlobalStateManager.is_fp8_calibration()
        self.fp8_meta["fp8_checkpoint"] = self.fp8 or self.fp8_calibration or self.fp8_meta["fp8_checkpoint"]
        if not (self.fp8 or self.fp8_calibration):
            return
        recipe = FP8GlobalStateManager.get_fp8_recipe()
        cur = self.fp8_meta.get("recipe")
        same = self.fp8_initialized and cur is not None and type(cur) is type(recipe) and \
            self.fp8_meta.get("num_gemms") == num_gemms
        if same and recipe.delayed():
            same = cur.amax_history_len == recipe.amax_history_len
        elif same and cur is not recipe:
            # stateless recipes: the quantizers are a function of the recipe's fields, so another object of the same
            # class with other settings (formats, Hadamard transform, block shapes, ...) needs new quantizers
            try:
                same = bool(cur == recipe)
            except Exception:  # noqa: BLE001  (user recipe classes without a usable __eq__)
                same = False
        self.fp8_meta["recipe"] = recipe
        self.fp8_meta["num_gemms"] = num_gemms
        if same:
            # keep states, but follow changes of margin/format made on a new recipe object
            for st in self._states.values():
                if st is not None:
                    st.recipe = recipe
            return
        dev = self._param_device()
        self._states["scaling_fwd"] = RecipeState.create(recipe, mode="forward", num_quantizers=3 * num_gemms, device=dev)
        self._states["scaling_bwd"] = RecipeState.create(recipe, mode="backward", num_quantizers=2 * num_gemms, device=dev)
        self.quantizers["scaling_fwd"] = self._states["scaling_fwd"].make_quantizers()
        self.quantizers["scaling_bwd"] = self._states["scaling_bwd"].make_quantizers()
        self._weight_cache.clear()
        self.fp8_initialized = True
        pending = self.fp8_meta.pop("_loaded_state", None)
        if pending is not None:
            self._apply_loaded_state(pending)

    def backward_override(self) -> Optional[str]:
        """``recipe.backward_override`` of the active recipe (None, ``"high_precision"`` or ``"dequantized"``).
        Modules that implement it run their backward GEMMs unquantized; the others refuse it."""
        recipe = self.fp8_meta.get("recipe")
        return getattr(recipe, "backward_override", None) if recipe is not None else None

    def _refuse_backward_override(self) -> None:
        if self.fp8 and self.backward_override() is not None:
            raise NotImplementedError(f"recipe.backward_override={self.backward_override()!r} is implemented by "
                                      f"Linear, LayerNormLinear and LayerNormMLP, not by {type(self).__name__}")

    def __getstate__(self):
        # the initialisers are closures (not picklable); a module restored from a pickle keeps its values and can
        # not be re-initialised
        state = self.__dict__.copy()
        state.pop("_init_fns", None)
        return state

    # ------------------------------------------------------------------ deferred initialisation
    def _param_init_fns(self) -> Dict[str, Any]:
        """``{parameter name: in-place initialiser}`` of this module's parameters (set by the constructors)."""
        return getattr(self, "_init_fns", {})

    def reset_parameters(self, defer_init: bool = False) -> None:
        """(Re-)initialise the parameters.  Parameters that were created on the ``meta`` device (``device="meta"``:
        construction without memory, as FSDP and checkpoint loaders want) are materialised first, on the GPU when
        there is one; the weights then get the module's ``init_method``, biases zeros, norm weights their identity
        value, and parameters created under ``quantized_model_init`` are quantized from the fresh values.
        (Reference: ``module/base.py`` ``reset_parameters``.)"""
        if defer_init:
            return
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        for name, fn in self._param_init_fns().items():
            p = getattr(self, name, None)
            if p is None:
                continue
            if isinstance(p, QuantizedTensorStorage):
                hp = torch.empty(tuple(p.shape), dtype=p.dtype, device=p.device)
                with torch.no_grad():
                    fn(hp)
                    p.quantize_(hp)
                continue
            if p.device.type == "meta":
                new = torch.nn.Parameter(torch.empty(tuple(p.shape), dtype=p.dtype, device=dev),
                                         requires_grad=p.requires_grad)
                for attr in ("tensor_model_parallel", "partition_dim", "partition_stride", "sequence_parallel"):
                    if hasattr(p, attr):
                        setattr(new, attr, getattr(p, attr))
                self.register_parameter(name, new)
                p = new
            with torch.no_grad():
                fn(p)
        if hasattr(self, "_fused_weight_storage"):
            views = [getattr(self, n) for n in getattr(self, "weight_names", [])]
            st = self._fused_weight_storage
            if st is not None and (st.device.type == "meta" or any(v.device != st.device for v in views)):
                self._fused_weight_storage = None      # the materialised parameters are separate tensors now
        pending = getattr(self, "_deferred_quantize", None)
        if pending:
            self._deferred_quantize = None
            self._quantize_primary_weights(pending)
        self._weight_cache.clear()

    def _quantize_primary_weights(self, weight_names) -> None:
        """``quantized_model_init``: replace the named high-precision weights by quantized parameters (both copies,
        so that forward, dgrad and wgrad read the parameter's own payload).  The quantizers come from a recipe state
        of their own: they describe how the PARAMETER is stored, whatever recipe later forward passes run under."""
        from ..quantization import RecipeState

        if any(getattr(self, n).device.type == "meta" for n in weight_names):
            # nothing to quantize yet: done by reset_parameters once the weights exist
            self._deferred_quantize = list(weight_names)
            self._model_init_recipe = FP8GlobalStateManager.FP8_MODEL_INIT_RECIPE
            return
        recipe = getattr(self, "_model_init_recipe", None) or FP8GlobalStateManager.FP8_MODEL_INIT_RECIPE
        st = RecipeState.create(recipe, mode="forward", num_quantizers=3, device=self._param_device())
        self._primary_state = st
        q = st.make_quantizers()[1]
        q.internal = False
        for n in weight_names:
            w = getattr(self, n)
            hp = w.detach()
            qt = q.copy()(hp) if hasattr(q, "copy") else q(hp)
            p = torch.nn.Parameter(qt)
            if self.preserve_high_precision_init_val:
                # kept on the host until the optimizer has built its master weights from it
                # (reference: module/base.py, get_/clear_high_precision_init_val on the parameter)
                p._high_precision_init_val = hp.cpu().clone()
                p.get_high_precision_init_val = (lambda p=p: getattr(p, "_high_precision_init_val", None))
                p.clear_high_precision_init_val = (lambda p=p: p.__dict__.pop("_high_precision_init_val", None) and None)
            for attr in ("tensor_model_parallel", "partition_dim", "partition_stride", "sequence_parallel"):
                if hasattr(w, attr):
                    setattr(p, attr, getattr(w, attr))
            self.register_parameter(n, p)

    def _param_device(self):
        for p in self.parameters(recurse=False):
            return p.device
        for p in self.parameters():
            return p.device
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")

    def prepare_forward(self, num_gemms: int = 1) -> None:
        self.init_fp8_metadata(num_gemms)
        st = self._states["scaling_fwd"]
        if self.fp8:
            # a custom recipe whose factory asked for delayed scaling: its amax histories are reduced and turned
            # into scales at region exit like those of the DelayedScaling recipe
            for key, fwd in (("scaling_fwd", True), ("scaling_bwd", False)):
                inner = getattr(self._states.get(key), "delayed", None)
                if inner is not None and (fwd or torch.is_grad_enabled()):
                    FP8GlobalStateManager.add_pending(inner, forward=fwd)
        if self.fp8 and isinstance(st, DelayedScalingRecipeState):
            from ..parallel import distributed as D

            if D.is_in_recompute() and self._recompute_scales:
                # second run of a checkpointed region: quantize with the scales of the first run, and put
                # the live scales and the amax slot back afterwards (the recompute records nothing new)
                old = self._recompute_scales.pop(0)
                live_scale, live_amax = st.scale.clone(), st.amax_history[0].clone()
                st.scale.copy_(old)

                def restore(st=st, live_scale=live_scale, live_amax=live_amax):
                    st.scale.copy_(live_scale)
                    st.amax_history[0].copy_(live_amax)

                D.add_recompute_restore(restore)
                if torch.is_grad_enabled():
                    FP8GlobalStateManager.add_pending(self._states["scaling_bwd"], forward=False)
                return
            if D.in_checkpoint_forward():
                self._recompute_scales.append(st.scale.clone())
            FP8GlobalStateManager.add_pending(st, forward=True)
            if torch.is_grad_enabled():
                FP8GlobalStateManager.add_pending(self._states["scaling_bwd"], forward=False)

    def get_quantizer(self, fwd: bool, idx: int) -> Optional[Quantizer]:
        if not self.fp8:
            return None
        q = self.quantizers["scaling_fwd" if fwd else "scaling_bwd"][idx]
        from .. import debug

        if debug.is_enabled():
            q = debug.wrap_quantizer(q, getattr(self, "name", None), fwd, idx)
        return q

    # ------------------------------------------------------------------ weights
    def get_quantized_weight(self, weight: torch.Tensor, quantizer: Optional[Quantizer], *, cache_name: str,
                             is_first_microbatch: Optional[bool] = None, need_columnwise: bool = True):
        """Quantize ``weight`` (both copies) or return the cached result.

        The cache is valid while the parameter has not changed: same torch version
        counter and same optimizer epoch; ``is_first_microbatch=False`` forces reuse
        and ``True`` forces an update, as in the reference.
        """
        if quantizer is None:
            return weight
        if isinstance(weight, QuantizedTensorStorage):
            if need_columnwise and hasattr(weight, "ensure_columnwise"):
                weight.ensure_columnwise()
            return weight
        quantizer.set_usage(rowwise=True, columnwise=need_columnwise)
        quantizer.internal = True
        key = (weight._version, weights_epoch(), need_columnwise, id(quantizer))
        ent = self._weight_cache.get(cache_name)
        if ent is not None and (is_first_microbatch is not True or _FREEZE_WEIGHT_CACHE[0]):
            if is_first_microbatch is False or ent[0] == key or _FREEZE_WEIGHT_CACHE[0]:
                if not need_columnwise or ent[1].get_usages()["columnwise"]:
                    return ent[1]
        q = quantizer(weight.detach())
        self._weight_cache[cache_name] = (key, q, weight, quantizer)
        return q

    def reset_weight_cache(self) -> None:
        self._weight_cache.clear()

    def requantize_cached_weights(self) -> None:
        """Quantize every cached weight again INTO its existing storage, so that kernels recorded in a
        CUDA graph (which hold those addresses) see the new values."""
        for name, (key, q, weight, quantizer) in list(self._weight_cache.items()):
            if weight is None:      # derived entries (stacked operands of grouped layers): rebuilt on next use
                del self._weight_cache[name]
                continue
            quantizer.set_usage(rowwise=True, columnwise=q.get_usages()["columnwise"])
            quantizer.internal = True
            quantizer.update_quantized(weight.detach(), q)
            self._weight_cache[name] = ((weight._version, weights_epoch()) + tuple(key[2:]), q, weight, quantizer)

    # ------------------------------------------------------------------ checkpoint
    def get_extra_state(self) -> torch.Tensor:
        """uint8 tensor with a pickle of the recipe and (delayed scaling) its scale/amax tensors."""
        if not self.fp8_meta.get("fp8_checkpoint") or self.fp8_meta.get("recipe") is None:
            return torch.empty(0, dtype=torch.uint8)
        recipe: Recipe = self.fp8_meta["recipe"]
        state: Dict[str, Any] = {"recipe": recipe}
        if recipe.delayed():
            f, b = self._states["scaling_fwd"], self._states["scaling_bwd"]
            if f is None:
                return torch.empty(0, dtype=torch.uint8)
            state["scale_fwd"] = f.scale.detach().cpu().clone()
            state["amax_history_fwd"] = f.amax_history.detach().cpu().clone()
            state["scale_bwd"] = b.scale.detach().cpu().clone()
            state["amax_history_bwd"] = b.amax_history.detach().cpu().clone()
        elif recipe.stateless():
            return torch.empty(0, dtype=torch.uint8)
        state["extra_fp8_variables"] = {
            k: v for k, v in self.fp8_meta.items()
            if isinstance(v, (bool, int, float, str)) and not k.startswith("_")
        }
        buf = io.BytesIO()
        pickle.dump(state, buf)
        return torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8).clone()

    def set_extra_state(self, state) -> None:
        if state is None:
            return
        import os

        if isinstance(state, torch.Tensor):
            if state.numel() == 0:
                return
            raw = bytes(state.detach().cpu().numpy().tobytes())
        elif isinstance(state, io.BytesIO):
            state.seek(0)
            raw = state.read()
        else:
            raise RuntimeError("Unsupported checkpoint format.")
        from ..utils.config import get_config

        if get_config().allow_unsafe_pickle_extra_state or os.getenv(_UNSAFE_PICKLE_ENV, "0") == "1":
            obj = pickle.loads(raw)
        else:
            obj = _SafeUnpickler(io.BytesIO(raw)).load()
        if obj is None:
            return
        if "recipe" not in obj:  # files written before recipes were stored
            obj["recipe"] = DelayedScaling()
        self.fp8_meta["fp8_checkpoint"] = True
        self.fp8_meta.update(obj.get("extra_fp8_variables", {}))
        if self.fp8_initialized and type(self.fp8_meta.get("recipe")) is type(obj["recipe"]):
            self._apply_loaded_state(obj)
        else:
            self.fp8_meta["_loaded_state"] = obj
            self.fp8_meta["recipe"] = obj["recipe"]

    def _apply_loaded_state(self, obj) -> None:
        recipe = obj["recipe"]
        if not recipe.delayed() or "scale_fwd" not in obj:
            return
        f, b = self._states["scaling_fwd"], self._states["scaling_bwd"]
        if not isinstance(f, DelayedScalingRecipeState):
            return

        def load(dst, src):
            if dst.shape != src.shape:
                warnings.warn(f"_extra_state shape mismatch {tuple(src.shape)} vs {tuple(dst.shape)}; "
                              "copying the overlapping part")
                sl = tuple(slice(0, min(a, c)) for a, c in zip(dst.shape, src.shape))
                dst[sl].copy_(src[sl])
            else:
                dst.copy_(src)

        load(f.scale, obj["scale_fwd"])
        load(f.amax_history, obj["amax_history_fwd"])
        load(b.scale, obj["scale_bwd"])
        load(b.amax_history, obj["amax_history_bwd"])

    # ------------------------------------------------------------------ delayed wgrad
    def backward_dw(self) -> None:
        """Run the weight-gradient GEMMs that were postponed with ``delay_wgrad_compute``."""
        if self.wgrad_store is not None:
            self.wgrad_store.pop()

    def need_backward_dw(self) -> bool:
        return self.wgrad_store is not None and self.wgrad_store.delay


class WeightGradStore:
    """Queue of postponed weight-gradient computations (zero-bubble pipeline schedules)."""

    def __init__(self, delay: bool = False) -> None:
        self.delay = delay
        self._queue: List = []

    def delay_wgrad_compute(self) -> bool:
        return self.delay

    def put(self, fn) -> None:
        self._queue.append(fn)

    def pop(self) -> None:
        q, self._queue = self._queue, []
        for fn in q:
            fn()


# communicator registry queries under the reference's names (``module/base.py``)
from ..parallel.comm_gemm import destroy_ub, initialize_ub, is_ub_initialized  # noqa: E402,F401
