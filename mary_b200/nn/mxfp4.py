"""MXFP4 names (src/nn/mxfp4.rs:257-361); the implementation lives in :mod:`mary_b200.nn.fp4`."""
from .fp4 import SpanError, decode_mxfp4, decode_nvfp4, e8m0_decode, quantize_mxfp4, transcode_mxfp4_to_nvfp4

transcode_to_nvfp4 = transcode_mxfp4_to_nvfp4
__all__ = ["SpanError", "decode_mxfp4", "decode_nvfp4", "e8m0_decode", "quantize_mxfp4", "transcode_mxfp4_to_nvfp4",
           "transcode_to_nvfp4"]
