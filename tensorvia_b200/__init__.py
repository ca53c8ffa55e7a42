"""tensorvia_b200 — a B200 (sm_100a) implementation of Tensorvia's matmul operator.

`ops.matmul` / `ops.Mul` is the operator; `_lib` is the ctypes view of the C ABI
(include/tvb.h) that a host program in any language binds to.  The CUDA library is
required: the first use of `ops`, `matmul`, `Mul`, `matmul_host` or `_lib` loads
`lib/libtvb.so` and raises if it has not been built (`python -m tensorvia_b200.build`).
Only the `build` submodule works without it.
"""
import importlib

__all__ = ["ops", "matmul", "Mul", "matmul_host", "sharded"]


def __getattr__(name):
    if name in ("ops", "_lib", "sharded"):
        return importlib.import_module(f"{__name__}.{name}")
    if name in ("matmul", "Mul", "matmul_host", "contiguous", "Slice", "Concat", "Transpose", "Typecast"):
        return getattr(importlib.import_module(f"{__name__}.ops"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
