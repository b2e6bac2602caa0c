"""B200-native paged attention for MLcompiler's continuous-batching path.

The product is the C-ABI shared library `libmlc_b200.so` (CUDA for sm_100a,
declared in include/mlc_b200.h). This package loads it through ctypes and
mirrors the reference's device-API member names on top of it; it contains no
CPU implementation of anything the kernels compute.
"""
from .capi import Executor, MlcError, load_library, library_path  # noqa: F401

__all__ = ["Executor", "MlcError", "load_library", "library_path"]
