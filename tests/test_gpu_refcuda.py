"""The reference's OWN CUDA backend, compiled for sm_100 from its sources (`make -C oracle refcuda`)
and run on this GPU in a process of its own (oracle/refcuda_run.py), as a second checker:

  * it pins the CUDA semantics of the restatement (oracle/matmul_oracle.c: tvo_matmul_cuda) — result
    dtypes of the CUDA backend (half x half -> half) and its accumulation — with outputs of the
    reference's real kernel instead of an argument from its source;
  * this repository's kernels are compared with it directly, at the usual bars.

Skipped where the library was not built (it is built where the reference tree is mounted and
travels as a binary)."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import refcheck as R
from gpuutil import Dev, assert_matches

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "oracle" / "_ref" / "libtv_ref_cuda.so"
F = lambda dt: 0 if dt >= R.BFLOAT16 else 1

CASES = [  # (dtype a, dtype b, shape a, shape b)
    (R.BFLOAT16, R.BFLOAT16, (300, 256), (256, 520)),
    (R.FLOAT16, R.FLOAT16, (2, 130, 128), (2, 128, 264)),
    (R.INT8, R.INT8, (257, 512), (512, 272)),
    (R.FLOAT32, R.FLOAT32, (200, 520), (520, 260)),
    (R.INT8, R.FLOAT16, (96, 64), (64, 80)),
    (R.BFLOAT16, R.FLOAT16, (70, 33), (33, 129)),
    (R.INT32, R.INT32, (65, 40), (40, 50)),
    # FLOAT64 results only with rows == cols: for them the reference launches its kernel with
    # `rows` in the place of `cols` (src/backend/cuda/mul.cu:91), which reads and writes out of
    # bounds for any other shape; such a shape is never run here
    (R.INT64, R.FLOAT32, (32, 17), (17, 32)),
    (R.FLOAT64, R.FLOAT64, (48, 40), (40, 48)),
    (R.INT16, R.INT8, (40, 24), (24, 31)),
]


def run_reference_cuda(dta, dtb, sa, sb, tmp_path, reps=1):
    out = tmp_path / "ref_cuda.npy"
    proc = subprocess.run([sys.executable, str(ROOT / "oracle" / "refcuda_run.py"), str(dta), str(dtb), "41", "42",
                           ",".join(map(str, sa)), ",".join(map(str, sb)), str(reps), str(out)],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    info = json.loads(proc.stdout.strip().splitlines()[-1])
    return np.load(out), info


@pytest.mark.skipif(not LIB.exists(), reason="reference CUDA backend not built (make -C oracle refcuda)")
@pytest.mark.parametrize("case", CASES)
def test_against_the_reference_cuda_backend(tv, tmp_path, case):
    dta, dtb, sa, sb = case
    ref_c, info = run_reference_cuda(dta, dtb, sa, sb, tmp_path)
    a = R.fill(sa, dta, 41, F(dta)); b = R.fill(sb, dtb, 42, F(dtb))
    # 1. the restatement of the CUDA semantics against the real CUDA backend
    exp, dte = R.oracle_matmul(a, dta, b, dtb, "cuda")
    assert dte == info["dtype_c"]
    if dte <= R.INT64:
        assert exp.tobytes() == ref_c.tobytes()
    else:
        tol = {R.BFLOAT16: 1e-2, R.FLOAT16: 1e-2, R.FLOAT32: 1e-6, R.FLOAT64: 1e-6}[dte]
        assert R.rel_frobenius(exp, ref_c, dte) <= tol
    # 2. this repository's kernels against the real CUDA backend
    dev = Dev(tv)
    try:
        c, dtc = dev.matmul(a, dta, b, dtb)
    finally:
        dev.free_all()
    tol64 = 1e-5 if dtc == R.FLOAT64 and R.INT64 in (dta, dtb) else 1e-12
    assert_matches(c, dtc, ref_c, info["dtype_c"], tol_f64=tol64, what=f"vs reference CUDA {case}")
