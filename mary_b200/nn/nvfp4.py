"""NVFP4 names (src/models/inkling/nvfp4.rs); the implementation lives in :mod:`mary_b200.nn.fp4`."""
from .fp4 import (E2M1, decode_nvfp4, e4m3_decode, e4m3_encode, quantize_act_nvfp4, quantize_weight_nvfp4,
                  swizzle_scales_128x4)

__all__ = ["E2M1", "decode_nvfp4", "e4m3_decode", "e4m3_encode", "quantize_act_nvfp4", "quantize_weight_nvfp4",
           "swizzle_scales_128x4"]
