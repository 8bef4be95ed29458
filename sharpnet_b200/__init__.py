"""sharpnet_b200: B200 (sm_100a) kernels behind SharpNet's Tensor.Dot / BatchMatrixMultiplication /
Dense-layer API.  The product is the C-ABI shared library built from ``csrc/``; the Python modules
mirror the reference's tensor and layer interface on top of it for tests and benchmarks."""
from ._capi import (ACT_CLIPPED_RELU, ACT_ELU, ACT_IDENTITY, ACT_LEAKY_RELU, ACT_LN, ACT_RELU, ACT_SIGMOID, ACT_SOFTMAX, ACT_SWISH, ACT_TANH, MATH_3XTF32, MATH_FP32_SIMT,  # noqa: F401
                    MATH_TF32, W_IN_OUT, W_OUT_IN, SharpNetB200Error)

__all__ = ["ACT_CLIPPED_RELU", "ACT_ELU", "ACT_IDENTITY", "ACT_LEAKY_RELU", "ACT_LN", "ACT_RELU", "ACT_SIGMOID", "ACT_SOFTMAX", "ACT_SWISH", "ACT_TANH", "MATH_3XTF32", "MATH_FP32_SIMT",
           "MATH_TF32", "W_IN_OUT", "W_OUT_IN", "SharpNetB200Error"]
