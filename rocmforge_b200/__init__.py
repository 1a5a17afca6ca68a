"""B200 (sm_100a) quantized-weight matmul path behind ROCmForge's operator surface.

The CUDA library (libb200q.so, C ABI in include/b200q.h) is the product; this package is the host-side
mirror of the reference's operator interface for that path. Importing the package does not load the
library; the first backend does, and raises if it was not built.
"""
from ._lib import (BF16, F32, LAYOUT_GGUF, LAYOUT_RF, MXFP4, MXFP6_E2M3, MXFP6_E3M2, ORIENT_KN, ORIENT_NK, Q4_0, Q4_K,  # noqa: F401
                   Q6_K, Q8_0, B200QError)

__all__ = ["B200QError", "Q4_0", "Q8_0", "Q4_K", "Q6_K", "MXFP4", "MXFP6_E2M3", "MXFP6_E3M2", "LAYOUT_RF", "LAYOUT_GGUF",
           "ORIENT_NK", "ORIENT_KN", "F32", "BF16"]
