"""onyxia_b200 — a B200-native execution backend for the Onyxia IR.

The product is the C-ABI library ``libonyxia_cuda.so`` (``include/onyxia_cuda.h``);
this package holds its sources (``csrc/``), the build step and a thin ctypes
mirror of the reference's ``Backend``/``Session`` interface used by the tests
and the benchmark.
"""
from . import ir  # noqa: F401
from ._ffi import OnyxiaError  # noqa: F401

__all__ = ["ir", "OnyxiaError"]
