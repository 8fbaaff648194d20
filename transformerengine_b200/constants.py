"""Enumerations and name tables shared by the front end (reference: ``pytorch/constants.py``).

``DType`` uses the numbering of the native launchers (``csrc/include/teb200/api.h`` / ``c_api.h``), extended with
the integer and 4-bit members the Python layer names; ``TE_DType`` maps torch dtypes to it."""
from __future__ import annotations

import enum

import torch


class DType(enum.IntEnum):
    kFloat32 = 0
    kFloat16 = 1
    kBFloat16 = 2
    kByte = 3
    kFloat8E4M3 = 4
    kFloat8E5M2 = 5
    kFloat4E2M1 = 6
    kInt32 = 7
    kInt64 = 8
    kFloat8E8M0 = 9   # scale bytes of MXFP8


TE_DType = {
    torch.uint8: DType.kByte,
    torch.int32: DType.kInt32,
    torch.int64: DType.kInt64,
    torch.float32: DType.kFloat32,
    torch.float16: DType.kFloat16,
    torch.bfloat16: DType.kBFloat16,
    torch.float8_e4m3fn: DType.kFloat8E4M3,
    torch.float8_e5m2: DType.kFloat8E5M2,
}
TE_DType_To_Torch = {v: k for k, v in TE_DType.items()}

AttnMaskTypes = ("no_mask", "padding", "causal", "padding_causal", "causal_bottom_right", "padding_causal_bottom_right",
                 "arbitrary")
AttnTypes = ("self", "cross")
AttnBiasTypes = ("pre_scale_bias", "post_scale_bias", "no_bias", "alibi")
QKVFormats = ("sbhd", "bshd", "thd")
LayerTypes = ("encoder", "decoder")
GemmParallelModes = ("row", "column", None)
dist_group_type = torch.distributed.ProcessGroup if torch.distributed.is_available() else object


class UserBufferQuantizationMode(enum.Enum):
    """Precision of the operands that travel through the fused collective GEMMs (``initialize_ub``)."""

    NONE = "none"
    FP8 = "fp8"
