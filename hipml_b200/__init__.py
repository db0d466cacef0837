"""B200 (sm_100a) implementation of hipml's full-attention hot path.

The product is ``lib/libhipml_cuda.so`` (C ABI in ``include/hipml_cuda.h``): KV
append/quantise, split-K decode over the q8_0 cache, multi-slot decode and causal chunk
prefill. ``api`` is a thin ctypes view of it for Python callers.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "api"]
