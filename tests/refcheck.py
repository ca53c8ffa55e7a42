"""Test-side access to the two CPU checkers (never imported by the product).

  oracle   oracle/libtv_oracle.so      our C restatement of the reference matmul
  ref      oracle/_ref/libtv_ref_cpu.so the reference library itself, built from its own
           sources by oracle/Makefile (present only where the reference tree was mounted
           at build time)

Arrays travel as raw element bits: bfloat16 as numpy uint16, float16 as numpy float16.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
ORACLE_LIB = ORACLE_DIR / "libtv_oracle.so"
REF_LIB = ORACLE_DIR / "_ref" / "libtv_ref_cpu.so"
GOLDEN_DIR = Path(__file__).resolve().parent / "golden"

INT8, INT16, INT32, INT64, BFLOAT16, FLOAT16, FLOAT32, FLOAT64 = range(8)
DTYPE_NAMES = ["int8", "int16", "int32", "int64", "bfloat16", "float16", "float32", "float64"]
NP = {INT8: np.int8, INT16: np.int16, INT32: np.int32, INT64: np.int64, BFLOAT16: np.uint16,
      FLOAT16: np.float16, FLOAT32: np.float32, FLOAT64: np.float64}

# seeds of the benchmark configurations: A = BASE + 2*cfg, B = BASE + 2*cfg + 1
SEED_BASE = 0x5EED0000


def build_oracle() -> Path:
    if not ORACLE_LIB.exists() or ORACLE_LIB.stat().st_mtime < (ORACLE_DIR / "matmul_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), "oracle"], check=True, capture_output=True)
    return ORACLE_LIB


_oracle = None
_ref = None


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        lib = C.CDLL(str(build_oracle()))
        i64, vp = C.c_int64, C.c_void_p
        lib.tvo_compute_type.restype = C.c_int
        lib.tvo_compute_type.argtypes = [C.c_int, C.c_int]
        for name in ("tvo_matmul_cpu", "tvo_matmul_cuda"):
            f = getattr(lib, name)
            f.restype = C.c_int
            f.argtypes = [vp, C.c_int, vp, C.c_int, vp, C.POINTER(C.c_int), i64, i64, i64, i64]
        lib.tvo_fill_splitmix.restype = C.c_int
        lib.tvo_fill_splitmix.argtypes = [vp, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int]
        lib.tvo_check_shapes.restype = C.c_int
        lib.tvo_check_shapes.argtypes = [C.c_int, C.POINTER(i64), C.c_int, C.POINTER(i64)]
        lib.tvo_threads.restype = C.c_int
        for name, src, dst in (("tvo_bf16_to_f32_n", np.uint16, np.float32), ("tvo_f16_to_f32_n", np.uint16, np.float32),
                               ("tvo_f32_to_bf16_n", np.float32, np.uint16), ("tvo_f32_to_f16_n", np.float32, np.uint16)):
            f = getattr(lib, name)
            f.restype = None
            f.argtypes = [vp, vp, C.c_size_t]
        _oracle = lib
    return _oracle


def have_ref() -> bool:
    return REF_LIB.exists()


def ref() -> C.CDLL:
    global _ref
    if _ref is None:
        # the reference prints a registration banner to stdout from a static initialiser
        # (src/factory.cpp:19, src/init.cpp:13); keep it off the caller's stdout
        sys.stdout.flush()
        saved = os.dup(1)
        devnull = os.open(os.devnull, os.O_WRONLY)
        try:
            os.dup2(devnull, 1)
            lib = C.CDLL(str(REF_LIB))
        finally:
            os.dup2(saved, 1)
            os.close(saved)
            os.close(devnull)
        i64p = C.POINTER(C.c_int64)
        lib.tvref_mul.restype = C.c_int
        lib.tvref_mul.argtypes = [C.c_void_p, C.c_int, C.c_int, i64p, C.c_void_p, C.c_int, C.c_int, i64p,
                                  C.c_void_p, C.c_uint64, C.POINTER(C.c_int), C.POINTER(C.c_int), i64p]
        lib.tvref_last_error.restype = C.c_char_p
        lib.tvref_compute_type.restype = C.c_int
        lib.tvref_compute_type.argtypes = [C.c_int, C.c_int]
        lib.tvref_threads.restype = C.c_int
        _ref = lib
    return _ref


# ---- conversions ------------------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    oracle().tvo_f32_to_bf16_n(x.ctypes.data, out.ctypes.data, x.size)
    return out


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    oracle().tvo_f32_to_f16_n(x.ctypes.data, out.ctypes.data, x.size)
    return out


def to_f64(arr: np.ndarray, dtype: int) -> np.ndarray:
    """Numeric value of a raw array as float64 (for error norms)."""
    if dtype == BFLOAT16:
        return bf16_bits_to_f32(arr).astype(np.float64)
    return arr.astype(np.float64)


def rel_frobenius(x: np.ndarray, ref_: np.ndarray, dtype: int) -> float:
    a, b = to_f64(x, dtype), to_f64(ref_, dtype)
    den = float(np.linalg.norm(b.ravel()))
    return float(np.linalg.norm((a - b).ravel())) / (den if den > 0 else 1.0)


# ---- seeded inputs ----------------------------------------------------------------------------
def fill(shape, dtype: int, seed: int, dist: int = 0, first: int = 0) -> np.ndarray:
    """Seeded synthetic tensor: floats uniform in [-1,1) (dist 0) or integers in [-10,10]."""
    arr = np.empty(shape, dtype=NP[dtype])
    rc = oracle().tvo_fill_splitmix(arr.ctypes.data, dtype, arr.size, seed, first, dist)
    assert rc == 0
    return arr


def splitmix_numpy(count: int, seed: int, first: int = 0) -> np.ndarray:
    """The generator restated in numpy: an independent check of the C and CUDA versions."""
    with np.errstate(over="ignore"):
        idx = np.arange(first + 1, first + count + 1, dtype=np.uint64)
        z = np.uint64(seed) + idx * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


# ---- running the checkers ------------------------------------------------------------------------
def _dims(shape):
    return (C.c_int64 * len(shape))(*shape)


def bmkn(shape_a, shape_b):
    if len(shape_a) == 3:
        return shape_a[0], shape_a[1], shape_a[2], shape_b[2]
    return 1, shape_a[0], shape_a[1], shape_b[1]


def oracle_matmul(a: np.ndarray, dta: int, b: np.ndarray, dtb: int, semantics: str = "cuda") -> tuple[np.ndarray, int]:
    """Runs the C restatement. semantics: "cuda" (mul.cu) or "cpu" (mul.cpp). -> (C, dtype)."""
    lib = oracle()
    batch, M, K, N = bmkn(a.shape, b.shape)
    if semantics == "cuda":
        dtc = lib.tvo_compute_type(dta, dtb)
    else:
        wa = FLOAT32 if dta in (BFLOAT16, FLOAT16) else dta
        wb = FLOAT32 if dtb in (BFLOAT16, FLOAT16) else dtb
        dtc = lib.tvo_compute_type(wa, wb)
    shape_c = (batch, M, N) if a.ndim == 3 else (M, N)
    c = np.empty(shape_c, dtype=NP[dtc])
    out_dt = C.c_int(-1)
    fn = lib.tvo_matmul_cuda if semantics == "cuda" else lib.tvo_matmul_cpu
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    rc = fn(a.ctypes.data, dta, b.ctypes.data, dtb, c.ctypes.data, C.byref(out_dt), batch, M, K, N)
    assert rc == 0, f"oracle failed rc={rc}"
    assert out_dt.value == dtc
    return c, dtc


def ref_matmul(a: np.ndarray, dta: int, b: np.ndarray, dtb: int) -> tuple[np.ndarray, int]:
    """Runs the reference library's own ops::Mul (CPU backend). -> (C, dtype). Raises RuntimeError
    with the reference's message when the reference throws."""
    lib = ref()
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    dtc, rank = C.c_int(-1), C.c_int(0)
    dims = (C.c_int64 * 3)()
    # first call sizes the result (c = NULL), second call fetches it
    rc = lib.tvref_mul(a.ctypes.data, dta, a.ndim, _dims(a.shape), b.ctypes.data, dtb, b.ndim, _dims(b.shape),
                       None, 0, C.byref(dtc), C.byref(rank), dims)
    if rc != 0:
        raise RuntimeError(lib.tvref_last_error().decode())
    shape_c = tuple(dims[i] for i in range(rank.value))
    c = np.empty(shape_c, dtype=NP[dtc.value])
    rc = lib.tvref_mul(a.ctypes.data, dta, a.ndim, _dims(a.shape), b.ctypes.data, dtb, b.ndim, _dims(b.shape),
                       c.ctypes.data, c.nbytes, C.byref(dtc), C.byref(rank), dims)
    if rc != 0:
        raise RuntimeError(lib.tvref_last_error().decode())
    return c, dtc.value


def ref_validate(shape_a, shape_b) -> str | None:
    """The reference's verdict on a pair of shapes: None if accepted, else its message."""
    a = np.zeros(int(np.prod(shape_a)), dtype=np.float32)
    b = np.zeros(int(np.prod(shape_b)), dtype=np.float32)
    lib = ref()
    dtc, rank = C.c_int(-1), C.c_int(0)
    dims = (C.c_int64 * 3)()
    rc = lib.tvref_mul(a.ctypes.data, FLOAT32, len(shape_a), _dims(shape_a), b.ctypes.data, FLOAT32,
                       len(shape_b), _dims(shape_b), None, 0, C.byref(dtc), C.byref(rank), dims)
    return None if rc == 0 else lib.tvref_last_error().decode()


def cuda_expected_from_cpu(c: np.ndarray, dtc_cpu: int, dta: int, dtb: int) -> tuple[np.ndarray, int]:
    """Turns a CPU-backend result into what the CUDA backend returns for the same inputs:
    same-type half inputs give a FLOAT32 result on the CPU and the half type on CUDA, so the
    fp32 result is rounded to nearest even."""
    if dta == dtb and dta == BFLOAT16:
        return f32_to_bf16_bits(c), BFLOAT16
    if dta == dtb and dta == FLOAT16:
        return f32_to_f16_bits(c).view(np.float16), FLOAT16
    return c, dtc_cpu


def sha(arr: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()
