"""Quantized tensor types and their quantizers."""
from .base import QuantizedTensor, QuantizedTensorStorage, Quantizer, prepare_for_saving, restore_from_saved
from .float8 import Float8Tensor, Float8TensorStorage, Float8Quantizer, Float8CurrentScalingQuantizer
from .mxfp8 import MXFP8Tensor, MXFP8TensorStorage, MXFP8Quantizer
from .nvfp4 import NVFP4Tensor, NVFP4TensorStorage, NVFP4Quantizer
from .blockwise import Float8BlockwiseQTensor, Float8BlockwiseQTensorStorage, Float8BlockQuantizer
from .hybrid import (HybridQuantizedTensor, HybridQuantizedTensorStorage, HybridQuantizer, IdentityQuantizer,
                     IdentityTensor, IdentityTensorStorage)
from .grouped import GroupedTensor, GroupedTensorStorage
