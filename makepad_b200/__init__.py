"""makepad_b200: B200-native block-quantised linear operators (libmpq) and a thin Python host mirror."""
from .quant_linear import (Context, MpqError, Nvfp4Weight, Q4Weight, QuantLinear, load_canonical, load_weight,  # noqa: F401
                           nvfp4_quantize, save_canonical, swiglu)
