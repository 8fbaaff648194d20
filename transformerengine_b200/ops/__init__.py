"""Functional ops.  Each op runs a hand-written sm_100a kernel for CUDA tensors and
the pure-PyTorch reference for CPU tensors.

The reference publishes its operation fuser under this name (``te.ops.Sequential``,
``te.ops.BasicLinear``, ... ``pytorch/ops/__init__.py``); those names resolve here too and
forward to :mod:`transformerengine_b200.fusible`.  The functional layer is also importable as
``transformerengine_b200.functional``."""
from . import _ext
from .quantize import (amax, quantize_fp8, dequantize_fp8, quantize_mxfp8, dequantize_mxfp8, quantize_nvfp4,
                       dequantize_nvfp4, swizzle_scales, unswizzle_scales)
from .quantize import hadamard_transform  # noqa: F401
from .gemm import gemm_nt, general_gemm, as_operand, Operand, set_mn_major_operands
from .norm import norm_fwd, norm_bwd
from .activation import activation_fwd, activation_bwd, is_gated
from .misc import (rope_apply, rope_qkv, rope_freqs, cross_entropy_fwd_bwd, cross_entropy_stats, cross_entropy_parallel_grad,
                   multi_tensor_adam, multi_tensor_sgd, multi_tensor_scale, multi_tensor_l2norm,
                   scaled_masked_softmax, softmax_bwd, dropout_fwd, dropout_bwd,
                   column_sum, splits_to_offsets, repad_rows, pad_last_dim, grouped_column_sum,
                   grouped_bias_add_, row_dot)
from .attention import attention, attention_ref, merge_attention_states


def check_status(device=None) -> None:
    """Raise if any kernel recorded a bounded-wait time-out since the last check."""
    import torch

    if not torch.cuda.is_available() or not _ext.available():
        return
    dev = torch.cuda.current_device() if device is None else device
    st = _ext.get().status(dev)
    code = int(st[0].item())
    if code != 0:
        st.zero_()
        names = {1: "producer wait", 2: "MMA wait", 3: "epilogue wait", 4: "peer flag wait", 5: "store wait",
                 6: "bad argument"}
        raise RuntimeError(f"device kernel reported status {code} ({names.get(code, 'unknown')})")


def __getattr__(name):
    """Fuser names (``Sequential``, ``BasicLinear``, ``FusibleOperation`` ...) looked up lazily: the fuser
    imports the modules, which import this package."""
    if name.startswith("__"):
        raise AttributeError(name)
    from .. import fusible

    if name in ("basic", "fused"):  # reference sub-packages: te.ops.basic.Bias, te.ops.fused.*
        return fusible
    if hasattr(fusible, name):
        return getattr(fusible, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
