"""tensorvia_b200 — a B200 (sm_100a) implementation of Tensorvia's matmul operator.

`ops.matmul` / `ops.Mul` is the operator; `_lib` is the ctypes view of the C ABI
(include/tvb.h) that a host program in any language binds to.  The CUDA library is
required: importing the package without `lib/libtvb.so` raises.
"""
from . import _lib, ops  # noqa: F401
from .ops import Mul, matmul, matmul_host  # noqa: F401

__all__ = ["ops", "matmul", "Mul", "matmul_host"]
