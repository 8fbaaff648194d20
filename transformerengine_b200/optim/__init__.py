from .fused_adam import FusedAdam, FusedSGD, multi_tensor_applier
