"""The modules under the reference's package name (``pytorch/module``)."""
from ..modules.base import TransformerEngineBaseModule, get_default_init_method  # noqa: F401
from ..modules.grouped_linear import Fp8Padding, Fp8Unpadding, GroupedLinear  # noqa: F401
from ..modules.layernorm_linear import LayerNorm, LayerNormLinear, RMSNorm  # noqa: F401
from ..modules.layernorm_mlp import LayerNormMLP  # noqa: F401
from ..modules.linear import Linear  # noqa: F401
from ..parallel.comm_gemm import destroy_ub, initialize_ub  # noqa: F401
