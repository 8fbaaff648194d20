"""Quantization recipes.

The recipe objects select how tensors are quantized inside :func:`autocast`.
Names, fields and environment defaults follow the reference
(``transformer_engine/common/recipe/__init__.py:29-708``) so that user code and
pickled ``_extra_state`` blobs written by either library can be read by the
other.  The classes report ``transformer_engine.common.recipe`` as their
module when pickled (see :func:`_install_pickle_alias`).
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, NamedTuple, Optional, Union


class _FormatHelper(NamedTuple):
    """Largest finite magnitude representable in the forward / backward dtype."""

    max_fwd: float
    max_bwd: float


class Format(Enum):
    """Low-precision number formats.

    ``HYBRID`` uses E4M3 for forward tensors and E5M2 for gradients.
    """

    E2M1 = _FormatHelper(max_fwd=6.0, max_bwd=6.0)
    E4M3 = _FormatHelper(max_fwd=448.0, max_bwd=448.0)
    E5M2 = _FormatHelper(max_fwd=57344.0, max_bwd=57344.0)
    HYBRID = _FormatHelper(max_fwd=448.0, max_bwd=57344.0)


@dataclass(frozen=True)
class MMParams:
    """Matmul options.  tcgen05 always accumulates in fp32 inside TMEM, so
    ``use_split_accumulator`` is accepted for compatibility only."""

    use_split_accumulator: bool = True


@dataclass(frozen=True)
class QParams:
    """Per-tensor-role quantization options."""

    power_2_scale: bool = False
    amax_epsilon: float = 0.0
    random_hadamard_transform: bool = False
    stochastic_rounding: bool = False
    fp4_2d_quantization: bool = False


def _env_flag(name: str, default: str = "0") -> bool:
    return os.getenv(name, default) == "1"


class Recipe:
    """Base class of all recipes."""

    def nvfp4(self) -> bool:
        return isinstance(self, NVFP4BlockScaling)

    def mxfp8(self) -> bool:
        return isinstance(self, MXFP8BlockScaling)

    def delayed(self) -> bool:
        return isinstance(self, DelayedScaling)

    def float8_current_scaling(self) -> bool:
        return isinstance(self, Float8CurrentScaling)

    def float8_per_tensor_scaling(self) -> bool:
        return isinstance(self, (DelayedScaling, Float8CurrentScaling))

    def float8_block_scaling(self) -> bool:
        return isinstance(self, Float8BlockScaling)

    def custom(self) -> bool:
        return isinstance(self, CustomRecipe)

    def stateless(self) -> bool:
        """True when the recipe carries no tensors between steps."""
        return not self.delayed()


@dataclass(repr=False)
class DelayedScaling(Recipe):
    """Per-tensor FP8 with scales derived from an amax history of earlier steps."""

    margin: int = 0
    fp8_format: Format = Format.HYBRID
    amax_history_len: int = 1024
    amax_compute_algo: Union[str, Callable] = "max"
    scaling_factor_compute_algo: Optional[Callable] = None
    reduce_amax: bool = True
    fp8_dpa: bool = False
    fp8_mha: bool = False
    backward_override: Optional[str] = field(
        default_factory=lambda: os.getenv("NVTE_BACKWARD_OVERRIDE", None)
    )

    def __post_init__(self) -> None:
        assert self.fp8_format != Format.E5M2, "Pure E5M2 training is not supported."
        assert self.amax_compute_algo in ("max", "most_recent") or callable(
            self.amax_compute_algo
        ), f"Unsupported amax_compute_algo {self.amax_compute_algo}"
        assert self.backward_override in (None, "high_precision", "dequantized")

    def __repr__(self) -> str:
        return (
            f"recipe_type={self.__class__.__name__}, margin={self.margin}, "
            f"format={str(self.fp8_format).split('.')[1]}, "
            f"amax_history_len={self.amax_history_len}, "
            f"reduce_amax={self.reduce_amax}, fp8_dpa={self.fp8_dpa}, fp8_mha={self.fp8_mha}"
        )


@dataclass(repr=False)
class Float8CurrentScaling(Recipe):
    """Per-tensor FP8 with the scale computed from the tensor being cast."""

    use_power_2_scales: bool = field(
        default_factory=lambda: _env_flag("NVTE_FP8_CURRENT_SCALING_POWER_2_SCALES")
    )
    fp8_format: Format = Format.HYBRID
    fp8_quant_fwd_inp: QParams = QParams(power_2_scale=False, amax_epsilon=0.0)
    fp8_quant_fwd_weight: QParams = QParams(power_2_scale=False, amax_epsilon=0.0)
    fp8_quant_bwd_grad: QParams = QParams(power_2_scale=False, amax_epsilon=0.0)
    fp8_gemm_fprop: MMParams = MMParams(use_split_accumulator=False)
    fp8_gemm_dgrad: MMParams = MMParams(use_split_accumulator=True)
    fp8_gemm_wgrad: MMParams = MMParams(use_split_accumulator=True)
    fp8_dpa: bool = False
    fp8_mha: bool = False
    backward_override: Optional[str] = field(
        default_factory=lambda: os.getenv("NVTE_BACKWARD_OVERRIDE", None)
    )

    def __post_init__(self) -> None:
        assert self.fp8_format != Format.E5M2, "Pure E5M2 training is not supported."

    def __repr__(self) -> str:
        return (
            f"recipe_type={self.__class__.__name__}, "
            f"format={str(self.fp8_format).split('.')[1]}, "
            f"use_power_2_scales={self.use_power_2_scales}"
        )


@dataclass(repr=False)
class MXFP8BlockScaling(Recipe):
    """FP8 data with one UE8M0 (power-of-two) scale per 32 consecutive values."""

    margin: int = 0
    fp8_format: Format = Format.E4M3
    fp8_dpa: bool = False
    fp8_mha: bool = False
    backward_override: Optional[str] = field(
        default_factory=lambda: os.getenv("NVTE_BACKWARD_OVERRIDE", None)
    )
    enable_2d_quantization: bool = False

    def __post_init__(self) -> None:
        assert self.fp8_format != Format.E5M2, "Pure E5M2 training is not supported."

    def __repr__(self) -> str:
        return (
            f"recipe_type={self.__class__.__name__}, margin={self.margin}, "
            f"format={str(self.fp8_format).split('.')[1]}"
        )


@dataclass(repr=False)
class Float8BlockScaling(Recipe):
    """FP8 data with fp32 scales per 1x128 (activations, gradients) or 128x128
    (weights) block."""

    use_f32_scales: bool = field(
        default_factory=lambda: _env_flag("NVTE_FP8_BLOCK_SCALING_FP32_SCALES")
    )
    fp8_format: Format = Format.E4M3
    fp8_quant_fwd_inp: QParams = QParams(power_2_scale=True, amax_epsilon=0.0)
    fp8_quant_fwd_weight: QParams = QParams(power_2_scale=True, amax_epsilon=0.0)
    fp8_quant_bwd_grad: QParams = QParams(power_2_scale=True, amax_epsilon=0.0)
    x_block_scaling_dim: int = 1
    w_block_scaling_dim: int = 2
    grad_block_scaling_dim: int = 1
    fp8_gemm_fprop: MMParams = MMParams(use_split_accumulator=True)
    fp8_gemm_dgrad: MMParams = MMParams(use_split_accumulator=True)
    fp8_gemm_wgrad: MMParams = MMParams(use_split_accumulator=True)
    fp8_dpa: bool = False
    fp8_mha: bool = False
    backward_override: Optional[str] = field(
        default_factory=lambda: os.getenv("NVTE_BACKWARD_OVERRIDE", None)
    )

    def __post_init__(self) -> None:
        assert self.x_block_scaling_dim in (1, 2)
        assert self.w_block_scaling_dim in (1, 2)
        assert self.grad_block_scaling_dim in (1, 2)
        assert not (
            self.x_block_scaling_dim == 2 and self.w_block_scaling_dim == 2
        ), "2D by 2D block scaling has no GEMM."
        if self.use_f32_scales:
            pow2 = False
        else:
            pow2 = True
        object.__setattr__(self, "fp8_quant_fwd_inp", QParams(power_2_scale=pow2))
        object.__setattr__(self, "fp8_quant_fwd_weight", QParams(power_2_scale=pow2))
        object.__setattr__(self, "fp8_quant_bwd_grad", QParams(power_2_scale=pow2))

    def __repr__(self) -> str:
        return (
            f"recipe_type={self.__class__.__name__}, "
            f"format={str(self.fp8_format).split('.')[1]}, "
            f"x_dim={self.x_block_scaling_dim}, w_dim={self.w_block_scaling_dim}, "
            f"grad_dim={self.grad_block_scaling_dim}"
        )


@dataclass(repr=False)
class NVFP4BlockScaling(Recipe):
    """E2M1 data, one E4M3 scale per 16 values and one fp32 scale per tensor.

    Defaults: activations 1D + random Hadamard transform on the transposed copy,
    weights 2D (16x16) without the transform, gradients 1D + transform +
    stochastic rounding (reference ``common/recipe/__init__.py:595-609``).
    """

    disable_rht: bool = field(default_factory=lambda: _env_flag("NVTE_NVFP4_DISABLE_RHT"))
    disable_stochastic_rounding: bool = field(
        default_factory=lambda: _env_flag("NVTE_NVFP4_DISABLE_STOCHASTIC_ROUNDING")
    )
    disable_2d_quantization: bool = field(
        default_factory=lambda: _env_flag("NVTE_NVFP4_DISABLE_2D_QUANTIZATION")
    )
    row_scaled_activation: bool = field(
        default_factory=lambda: _env_flag("NVTE_NVFP4_ROW_SCALED_ACTIVATION")
    )
    nvfp4_4over6: str = field(default_factory=lambda: os.getenv("NVTE_NVFP4_4OVER6", "none"))
    nvfp4_4over6_e4m3_use_256: str = field(default_factory=lambda: os.getenv("NVTE_NVFP4_4OVER6_E4M3_USE_256", "all"))
    nvfp4_4over6_err_mode: str = field(
        default_factory=lambda: os.getenv("NVTE_NVFP4_4OVER6_ERR_MODE", "MAE").upper())
    fp4_format: Format = Format.E2M1
    fp8_format: Format = Format.E4M3
    fp8_dpa: bool = False
    fp8_mha: bool = False
    backward_override: Optional[str] = field(
        default_factory=lambda: os.getenv("NVTE_BACKWARD_OVERRIDE", None)
    )
    fp4_quant_fwd_inp: QParams = field(default=None)  # type: ignore[assignment]
    fp4_quant_fwd_weight: QParams = field(default=None)  # type: ignore[assignment]
    fp4_quant_bwd_grad: QParams = field(default=None)  # type: ignore[assignment]

    def __post_init__(self) -> None:
        assert self.fp4_format == Format.E2M1
        assert self.fp8_format == Format.E4M3
        scopes = ("none", "weights", "activations", "all")
        assert self.nvfp4_4over6 in scopes, f"nvfp4_4over6 must be one of {scopes}"
        assert self.nvfp4_4over6_e4m3_use_256 in scopes, f"nvfp4_4over6_e4m3_use_256 must be one of {scopes}"
        self.nvfp4_4over6_err_mode = str(self.nvfp4_4over6_err_mode).upper()
        assert self.nvfp4_4over6_err_mode in ("MAE", "MSE"), "nvfp4_4over6_err_mode must be 'MAE' or 'MSE'"
        rht = not self.disable_rht
        self.fp4_quant_fwd_inp = QParams(
            random_hadamard_transform=rht, stochastic_rounding=False, fp4_2d_quantization=False
        )
        self.fp4_quant_fwd_weight = QParams(
            random_hadamard_transform=False,
            stochastic_rounding=False,
            fp4_2d_quantization=not self.disable_2d_quantization,
        )
        self.fp4_quant_bwd_grad = QParams(
            random_hadamard_transform=rht,
            stochastic_rounding=not self.disable_stochastic_rounding,
            fp4_2d_quantization=False,
        )

    def __repr__(self) -> str:
        return (
            f"recipe_type={self.__class__.__name__}, rht={not self.disable_rht}, "
            f"sr={not self.disable_stochastic_rounding}, "
            f"2d={not self.disable_2d_quantization}"
        )


@dataclass(repr=False)
class CustomRecipe(Recipe):
    """User-supplied quantizer factory: ``qfactory(role) -> Quantizer``.

    ``role`` is one of ``linear_input``, ``linear_weight``, ``linear_output``,
    ``linear_grad_output``, ``linear_grad_input``.
    """

    qfactory: Callable = None  # type: ignore[assignment]
    fp8_format: Format = Format.HYBRID
    fp8_dpa: bool = False
    fp8_mha: bool = False
    backward_override: Optional[str] = None
    quantization_alignment: int = 128

    def __repr__(self) -> str:
        return f"recipe_type={self.__class__.__name__}, qfactory={self.qfactory}"


_ALIAS = "transformer_engine.common.recipe"


def _install_pickle_alias() -> None:
    """Make recipe pickles portable between this library and the reference.

    Recipes are pickled inside ``_extra_state``.  The reference resolves them
    at ``transformer_engine.common.recipe``; when that package is not
    installed, this module is registered under the same dotted name, and the
    classes advertise that name so the bytes written here load there too.
    """
    import importlib.util
    import types

    try:
        real = importlib.util.find_spec("transformer_engine") is not None
    except (ImportError, ValueError):
        real = False
    me = sys.modules[__name__]
    if not real:
        root = sys.modules.setdefault("transformer_engine", types.ModuleType("transformer_engine"))
        common = sys.modules.setdefault(
            "transformer_engine.common", types.ModuleType("transformer_engine.common")
        )
        root.common = common  # type: ignore[attr-defined]
        common.recipe = me  # type: ignore[attr-defined]
        sys.modules.setdefault(_ALIAS, me)
        for cls in (
            Format,
            MMParams,
            QParams,
            Recipe,
            DelayedScaling,
            Float8CurrentScaling,
            MXFP8BlockScaling,
            Float8BlockScaling,
            NVFP4BlockScaling,
            CustomRecipe,
            _FormatHelper,
        ):
            cls.__module__ = _ALIAS


_install_pickle_alias()

__all__ = [
    "Format",
    "MMParams",
    "QParams",
    "Recipe",
    "DelayedScaling",
    "Float8CurrentScaling",
    "MXFP8BlockScaling",
    "Float8BlockScaling",
    "NVFP4BlockScaling",
    "CustomRecipe",
]
