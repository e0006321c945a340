"""B200-native attention hot path for YVEX (yailabs/clori): host-side mirror.

The product is libyvex_b200.so (C11 host layer + sm_100a CUDA kernels behind a
C-ABI). This package is a thin ctypes view of that ABI for tests, the benchmark
and Python callers; it computes nothing itself and has no fallback.
"""
from . import abi
from .operator import (Backend, KvPool, Tensor, YvexError, attention_requirement, bf16_bits_to_f32,
                       f32_to_bf16_bits)

__all__ = ["abi", "Backend", "KvPool", "Tensor", "YvexError", "attention_requirement",
           "bf16_bits_to_f32", "f32_to_bf16_bits"]
