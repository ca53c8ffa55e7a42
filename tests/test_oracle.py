"""The C restatement (oracle/matmul_oracle.c) against the golden fixtures, which are outputs
of the reference library itself (tests/golden/make_golden.py), and — where the reference
library is present — against the reference run live."""
import json

import numpy as np
import pytest

import refcheck as R

META = json.loads((R.GOLDEN_DIR / "golden_meta.json").read_text())
SMALL = np.load(R.GOLDEN_DIR / "golden_small.npz")
TILED = np.load(R.GOLDEN_DIR / "golden_tiled.npz")
CONFIGS = np.load(R.GOLDEN_DIR / "golden_configs.npz")
F = lambda dt: 0 if dt >= R.BFLOAT16 else 1


def test_compute_type_table():
    # via::compute_type, include/core/type_traits.h:270-287, as executed by the reference
    table = [[R.oracle().tvo_compute_type(a, b) for b in range(8)] for a in range(8)]
    assert table == META["compute_type"]
    assert table[R.BFLOAT16][R.BFLOAT16] == R.BFLOAT16 and table[R.FLOAT16][R.FLOAT16] == R.FLOAT16
    assert table[R.INT8][R.INT8] == R.INT8 and table[R.INT64][R.FLOAT16] == R.FLOAT64
    assert R.oracle().tvo_compute_type(8, 0) == -1


@pytest.mark.parametrize("a", range(8))
@pytest.mark.parametrize("b", range(8))
def test_small_path_all_pairs_bit_exact(a, b):
    A = R.fill((5, 7), a, 1000 + a, F(a)); B = R.fill((7, 6), b, 2000 + b, F(b))
    c, dt = R.oracle_matmul(A, a, B, b, "cpu")
    assert dt == int(SMALL[f"m2_{a}_{b}_dt"])
    assert c.tobytes() == SMALL[f"m2_{a}_{b}"].tobytes()
    A = R.fill((2, 3, 4), a, 3000 + a, F(a)); B = R.fill((2, 4, 5), b, 4000 + b, F(b))
    c, dt = R.oracle_matmul(A, a, B, b, "cpu")
    assert dt == int(SMALL[f"m3_{a}_{b}_dt"])
    assert c.tobytes() == SMALL[f"m3_{a}_{b}"].tobytes()


@pytest.mark.parametrize("name", sorted(META["tiled"]))
def test_tiled_path_bit_exact(name):
    m = META["tiled"][name]
    A = R.fill(tuple(m["shape_a"]), m["dta"], 5000 + m["dta"], F(m["dta"]))
    B = R.fill(tuple(m["shape_b"]), m["dtb"], 6000 + m["dtb"], F(m["dtb"]))
    assert R.sha(A) == m["sha_a"] and R.sha(B) == m["sha_b"], "seeded generator drifted"
    c, dt = R.oracle_matmul(A, m["dta"], B, m["dtb"], "cpu")
    assert dt == m["dtc"]
    flat = c.reshape(-1, c.shape[-1])
    assert flat[m["rows"]].tobytes() == TILED[f"{name}_rows"].tobytes()
    assert R.sha(c) == m["sha_c"]


@pytest.mark.parametrize("a,b", [(a, b) for a in range(8) for b in range(8)])
def test_cuda_semantics_agree_with_cpu_backend_on_small_outputs(a, b):
    """mul_cuda_3d and mul_kernel_basic share their arithmetic (promoted accumulator, k ascending);
    they differ only in the result dtype for same-type halves, where CUDA rounds the fp32 sum."""
    A = R.fill((5, 7), a, 1000 + a, F(a)); B = R.fill((7, 6), b, 2000 + b, F(b))
    c, dt = R.oracle_matmul(A, a, B, b, "cuda")
    exp, dte = R.cuda_expected_from_cpu(SMALL[f"m2_{a}_{b}"], int(SMALL[f"m2_{a}_{b}_dt"]), a, b)
    if dt == dte:
        assert c.tobytes() == exp.tobytes()
    else:
        # bf16 x f16 and half x int: CUDA result is FLOAT32 as on the CPU, values identical
        assert dt == R.oracle().tvo_compute_type(a, b)
        assert R.rel_frobenius(c, exp, dt) == 0.0


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_benchmark_config_rows(cfg):
    """Sampled rows of the five full-size configurations: oracle on the same rows of A."""
    from golden.make_golden import gen_rows
    m = META["configs"][str(cfg)]
    dt, K, N, M = m["dtype"], m["K"], m["N"], m["M"]
    kept = [tuple(p) for p in m["kept"]]
    gold = CONFIGS[f"c{cfg}_rows"]
    assert R.sha(gold) == m["sha_rows"]
    # keep the CPU suite short: check a few of the stored rows per configuration
    pick = list(range(0, len(kept), max(1, len(kept) // 3)))[:3]
    for i in pick:
        b, r = kept[i]
        a_row = gen_rows(dt, K, [(b, r)], M, m["seed_a"], m["dist"])
        Bm = R.fill((K, N), dt, m["seed_b"], m["dist"], first=b * K * N)
        # 1 x N output is far below 1 Mi: force the reference's tiled arithmetic by tiling the row
        # 64-chunk partial sums are what mul_kernel_tiled adds; restate that here directly
        if dt in (R.BFLOAT16, R.FLOAT16):
            af = R.bf16_bits_to_f32(a_row) if dt == R.BFLOAT16 else a_row.view(np.float16).astype(np.float32)
            bf = R.bf16_bits_to_f32(Bm) if dt == R.BFLOAT16 else Bm.astype(np.float32)
        else:
            af, bf = a_row, Bm
        big_a = np.repeat(af, 1024 * 1024 // N + 1, axis=0)   # enough identical rows for the tiled path
        src_dt = R.FLOAT32 if dt in (R.BFLOAT16, R.FLOAT16) else dt
        c, _ = R.oracle_matmul(big_a, src_dt, bf, src_dt, "cpu")
        assert c[0].tobytes() == gold[i].tobytes(), f"config {cfg} row {(b, r)}"


def test_shape_rules_match_reference_messages():
    for case in META["shape_messages"]:
        sa, sb = case["a"], case["b"]
        code = R.oracle().tvo_check_shapes(len(sa), (R.C.c_int64 * len(sa))(*sa), len(sb), (R.C.c_int64 * len(sb))(*sb))
        assert (code == 0) == (case["message"] is None), case


def test_half_conversions_exhaustive():
    # every f16 bit pattern widens like numpy; every widened value rounds back to itself
    bits = np.arange(65536, dtype=np.uint16)
    f = np.empty(65536, np.float32)
    R.oracle().tvo_f16_to_f32_n(bits.ctypes.data, f.ctypes.data, 65536)
    want = bits.view(np.float16).astype(np.float32)
    ok = (f == want) | (np.isnan(f) & np.isnan(want))
    assert ok.all()
    finite = np.isfinite(want)
    back = R.f32_to_f16_bits(want)
    assert (back[finite] == bits[finite]).all()
    # random fp32 values round to f16 / bf16 like numpy / like the textbook RNE
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * np.float32(s) for s in (1e-8, 1e-4, 1, 300, 70000)])
    with np.errstate(over="ignore"):
        assert (R.f32_to_f16_bits(x) == x.astype(np.float16).view(np.uint16)).all()
    u = x.view(np.uint32).astype(np.uint64)
    rne = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    assert (R.f32_to_bf16_bits(x) == rne).all()
    # halfway cases
    ties = np.array([0x3F808000, 0x3F818000, 0x3F800001 | 0x8000], dtype=np.uint32).view(np.float32)
    assert R.f32_to_bf16_bits(ties).tolist() == [0x3F80, 0x3F82, 0x3F81]


def test_seeded_generator_matches_numpy_restatement():
    u = R.splitmix_numpy(4096, 0x5EED0002, first=17)
    f = (u >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 8388608.0) - np.float32(1.0)
    assert (R.fill((4096,), R.FLOAT32, 0x5EED0002, 0, first=17) == f).all()
    assert f.min() >= -1.0 and f.max() < 1.0
    i = (u % np.uint64(21)).astype(np.int64) - 10
    assert (R.fill((4096,), R.INT8, 0x5EED0002, 1, first=17) == i).all()
    assert i.min() == -10 and i.max() == 10
    assert (R.fill((4096,), R.INT64, 0x5EED0002, 0, first=17) == i).all()
    assert (R.fill((4096,), R.BFLOAT16, 0x5EED0002, 0, first=17) == R.f32_to_bf16_bits(f)).all()
    assert (R.fill((4096,), R.FLOAT16, 0x5EED0002, 0, first=17).view(np.uint16) == R.f32_to_f16_bits(f)).all()
    # a slice regenerated on its own equals the slice of the whole
    whole = R.fill((1000,), R.FLOAT32, 7, 0)
    assert (R.fill((100,), R.FLOAT32, 7, 0, first=300) == whole[300:400]).all()


@pytest.mark.skipif(not R.have_ref(), reason="reference library not built on this machine")
def test_oracle_equals_live_reference_on_random_shapes():
    rng = np.random.default_rng(3)
    for _ in range(12):
        a, b = int(rng.integers(0, 8)), int(rng.integers(0, 8))
        M, K, N = (int(v) for v in rng.integers(1, 40, 3))
        A = R.fill((M, K), a, int(rng.integers(1, 1 << 30)), F(a)); B = R.fill((K, N), b, int(rng.integers(1, 1 << 30)), F(b))
        cr, dr = R.ref_matmul(A, a, B, b)
        co, do = R.oracle_matmul(A, a, B, b, "cpu")
        assert dr == do and cr.tobytes() == co.tobytes()
