"""B200-native (sm_100a) device runtime for the PolarAI builtin kernels.

The product is native: csrc/ holds the CUDA kernels and their C ABI
(include/polar_b200.h) and the device-runtime plugin that a PolarAI executor
loads (include/polar_b200_rt.h).  The Python modules are thin ctypes bindings
used by the tests and the benchmark; they never compute anything themselves and
raise if the CUDA library is missing.
"""
from .capi import Library, PolarB200Error, lib  # noqa: F401
