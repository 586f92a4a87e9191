"""ferrum_cpu_b200 — Ferrum's Q8_0 GPT-2 forward path on NVIDIA B200.

The product is libferrum_cuda.so (hand-written sm_100a CUDA behind the C ABI of
include/ferrum_cuda.h). This package holds its sources (csrc/), the build step, a ctypes
binding and a small Python mirror of the reference interfaces used by tests and benchmarks.
"""
from . import _lib, synth  # noqa: F401
from ._lib import (FC_MATH_BF16X3, FC_MATH_FP32, FerrumCudaError, LIB_PATH)  # noqa: F401
from .engine import (CudaSlm, QWeight, Score, device_count, gguf_probe, q8_0_linear, sample_logits, sampling,  # noqa: F401
                     take_launch_count)
