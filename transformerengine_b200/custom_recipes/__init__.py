"""Quantizer factories for ``recipe.CustomRecipe(qfactory=...)`` and a reference GEMM on quantized
operands (reference: ``pytorch/custom_recipes/``)."""
from .gemm import custom_gemm  # noqa: F401
from . import quantizer_factories, quantizer_factory_zoo  # noqa: F401
