"""Legacy module name of the quantization front end (reference: ``pytorch/fp8.py`` re-exports ``quantization``)."""
from .quantization import *  # noqa: F401,F403
from .quantization import (FP8GlobalStateManager, autocast, fp8_autocast, fp8_model_init,  # noqa: F401
                           get_default_fp8_recipe, is_fp8_available, quantized_model_init)
