"""candle_b200: B200 (sm_100a) implementation of candle's GGUF quantized-matmul path.

The work is done by ``lib/libcandle_q_b200.so`` (CUDA kernels + C++ host objects, C ABI in
``include/candle_q_b200.h``).  This Python package is only a binding for tests, benchmarks and model
glue: it hands torch device pointers and streams to the library.  There is no CPU or PyTorch fallback;
importing ``candle_b200.quantized`` without the built library raises.
"""
from .capi import CandleQError  # noqa: F401

__all__ = ["CandleQError"]
