"""B200-native NF4 quantized-linear hot path (quantize, dequantize, QLoRA forward).

The compute lives in ``libnf4b200.so`` (hand-written CUDA for sm_100a behind a C ABI,
see ``include/nf4_b200.h``); these modules mirror the reference crate's API names on top
of it.  Build the library with ``python -m unifur_b200.build``.
"""
from ._lib import (DTYPE_BF16, DTYPE_F32, LAYOUT_IN_OUT, LAYOUT_OUT_IN, Nf4Error,  # noqa: F401
                   launch_count)

__all__ = ["DTYPE_BF16", "DTYPE_F32", "LAYOUT_IN_OUT", "LAYOUT_OUT_IN", "Nf4Error",
           "launch_count"]
