"""fastconv_b200: B200-native (sm_100a) convolution-layer hot path behind FastConv's operator API.

The product is libfastconv_b200.so (hand-written CUDA behind the C ABI of include/fastconv_b200.h).
This package is the thin host-side mirror of the reference's ConvLayer interface used by the tests
and the benchmark; importing it never falls back to a CPU implementation.
"""
from . import synth  # noqa: F401
from ._lib import (ALGO_AUTO, ALGO_DIRECT, ALGO_IM2COL, ALGO_WINOGRAD, MATH_3XTF32, MATH_FP32_MIRRORED,  # noqa: F401
                   MATH_TF32, ConvDesc, FastConvError, load)
from .layers import (Context, ConvDirectLayer, ConvIm2colLayer, ConvLayer, ConvWinoF63ZCLayer, LayerList, default_context, diff,  # noqa: F401
                     make_desc, make_layer, output_size, resolve_plan, select_algorithm)

__all__ = [
    "Context", "LayerList", "ConvLayer", "ConvWinoF63ZCLayer", "ConvIm2colLayer", "ConvDirectLayer", "ConvDesc", "FastConvError", "make_desc",
    "make_layer", "output_size", "select_algorithm", "resolve_plan", "diff", "default_context", "load", "synth",
]
