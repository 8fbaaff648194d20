"""B200-native low-precision transformer library (PyTorch front end).

Public surface mirrors ``transformer_engine.pytorch``: the modules ``Linear``,
``LayerNormLinear``, ``LayerNormMLP``, ``GroupedLinear``, ``LayerNorm``,
``RMSNorm``, ``DotProductAttention``, ``MultiheadAttention``,
``TransformerLayer``; ``autocast`` / ``fp8_autocast`` with the recipes in
``transformerengine_b200.recipe``; ``quantized_model_init``; ``checkpoint``;
fused optimizers.  CUDA tensors run hand-written sm_100a kernels; CPU tensors run
a pure-PyTorch reference path with the same numerics.
"""
from .common import recipe  # noqa: F401
from . import ops  # noqa: F401
from . import ops as functional  # noqa: F401  (the functional layer under an unambiguous name)
from .ops import check_status  # noqa: F401
from . import tensor  # noqa: F401
from .quantization import (autocast, fp8_autocast, quantized_model_init, fp8_model_init, FP8GlobalStateManager,
                           is_fp8_available, is_mxfp8_available, is_nvfp4_available,
                           is_fp8_block_scaling_available, get_default_fp8_recipe, get_default_recipe)
from .modules.linear import Linear
from .modules.layernorm_linear import LayerNormLinear, LayerNorm, RMSNorm
from .modules.layernorm_mlp import LayerNormMLP
from .attention.dot_product_attention import DotProductAttention
from .attention.multi_head_attention import MultiheadAttention
from .attention.rope import RotaryPositionEmbedding, apply_rotary_pos_emb
from .attention.inference import InferenceParams, KVCacheManager, NonPagedKVCacheManager, PagedKVCacheManager
from .attention.fused_mla_q_uproj import FusedMLAQUpProjRopeQuant
from .attention import thd  # noqa: F401  packed-sequence helpers
from .transformer import TransformerLayer
from .modules.grouped_linear import GroupedLinear, Fp8Padding, Fp8Unpadding
from .moe import (fused_topk_with_score_function, fused_compute_score_for_moe_aux_loss, fused_moe_aux_loss,
                  moe_permute, moe_permute_with_probs, moe_permute_and_pad_with_probs, moe_unpermute,
                  moe_sort_chunks_by_index, moe_sort_chunks_by_index_with_probs)
from .ep import (ep_dispatch, ep_combine, ep_bootstrap, ep_finalize, ep_prepare, is_ep_bootstrapped,  # noqa: F401
                 is_symm_backed, EpBuffer)
from .parallel.distributed import checkpoint, CudaRNGStatesTracker
from .optim import FusedAdam, FusedSGD
from .parallel.comm_gemm import initialize_ub, destroy_ub
from . import optimizers  # noqa: F401  (the reference's package name; implementations in optim/)
from . import fusible  # noqa: F401  (operation fuser: fusible.Sequential and the basic operations)
from . import debug  # noqa: F401
from .graph import make_graphed_callables
from .cpu_offload import get_cpu_offload_context
from .export import onnx_export, is_in_onnx_export_mode
from .cross_entropy import parallel_cross_entropy
from .newton_schulz import newton_schulz, CusolverMpCtx
from .parallel.context_parallel import (get_batch_on_this_cp_rank, pad_thd_sequences_for_cp,  # noqa: F401
                                        generate_positional_ids_for_cp)

# names that reference code imports from the top level of the package
from . import constants  # noqa: F401
from .constants import DType, UserBufferQuantizationMode  # noqa: F401
from .quantization import QuantizerRole, QuantizerRequest, DelayedScalingRequest  # noqa: F401
from .tensor import (Quantizer, QuantizedTensor, QuantizedTensorStorage, Float8Quantizer,  # noqa: F401
                     Float8CurrentScalingQuantizer, Float8Tensor, Float8TensorStorage, MXFP8Quantizer, MXFP8Tensor,
                     MXFP8TensorStorage, NVFP4Quantizer, NVFP4Tensor, NVFP4TensorStorage, Float8BlockQuantizer,
                     Float8BlockwiseQTensor, Float8BlockwiseQTensorStorage)
from .tensor.hybrid import (HybridQuantizer, HybridQuantizedTensor, HybridQuantizedTensorStorage,  # noqa: F401
                            IdentityQuantizer, IdentityTensor, IdentityTensorStorage)
from .tensor.base import prepare_for_saving, restore_from_saved, restore_from_func_ctx  # noqa: F401
# unpickling entry points of the quantized tensor classes (pickles written by this library name them)
from .tensor.float8 import _make_float8_tensor_in_reduce_ex  # noqa: F401
from .tensor.mxfp8 import _make_mxfp8_tensor_in_reduce_ex  # noqa: F401
from .tensor.nvfp4 import _make_nvfp4_tensor_in_reduce_ex  # noqa: F401
from .tensor.blockwise import _make_blockwise_in_reduce_ex as _make_float8_blockwise_tensor_in_reduce_ex  # noqa: F401
from .tensor.hybrid import _make_identity_tensor_in_reduce_ex  # noqa: F401
from .tensor.hybrid import _make_hybrid_tensor_in_reduce_ex as _make_hybrid_quantized_tensor_in_reduce_ex  # noqa: F401
from .cpu_offload import ManualOffloadSynchronizer, mark_not_offload  # noqa: F401
from .utils import (get_device_compute_capability, get_cudnn_version, is_bf16_available, torch_version,  # noqa: F401
                    interleave_glu_tensor, deinterleave_glu_tensor)


def load_framework_extension(framework: str = "torch") -> None:
    """Load (building it first if needed) the native extension; only the PyTorch front end exists."""
    if framework not in ("torch", "pytorch"):
        raise ValueError(f"no {framework} front end in this library")
    from .ops import _ext

    _ext.get()


__version__ = "0.1.0"

from . import compat  # noqa: E402,F401
import os as _os  # noqa: E402

if _os.environ.get("TEB200_ALIAS_TRANSFORMER_ENGINE", "0") == "1":
    compat.install_as_transformer_engine()
