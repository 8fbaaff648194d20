"""Storage classes of the quantized tensors under the reference's package name (``pytorch/tensor/storage``)."""
from ..blockwise import Float8BlockwiseQTensorStorage  # noqa: F401
from ..float8 import Float8TensorStorage  # noqa: F401
from ..grouped import GroupedTensorStorage  # noqa: F401
from ..hybrid import HybridQuantizedTensorStorage, IdentityTensorStorage  # noqa: F401
from ..mxfp8 import MXFP8TensorStorage  # noqa: F401
from ..nvfp4 import NVFP4TensorStorage  # noqa: F401
