"""Base classes of the quantized tensors under the reference's module name (``pytorch/quantized_tensor.py``)."""
from .tensor.base import (QuantizedTensor, QuantizedTensorStorage, Quantizer, prepare_for_saving,  # noqa: F401
                          restore_from_func_ctx, restore_from_saved)
