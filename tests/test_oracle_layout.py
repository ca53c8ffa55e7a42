"""The C restatement of the layout operations (oracle/layout_oracle.c) against the golden
fixtures, which are outputs of the reference library itself (tests/golden/make_golden.py), and —
where the reference library is present — against the reference run live.  Byte moves: bit-exact."""
import numpy as np
import pytest

import refcheck as R
from layout_cases import (CONCAT_CASES, LAYOUT_DTYPES, MUL_VIEW_CASES, PERMUTE_CASES, SLICE_CASES,
                          pinned_casts, pins_view_route, typecast_input)

GOLD = np.load(R.GOLDEN_DIR / "golden_layout.npz")
F = lambda dt: 0 if dt >= R.BFLOAT16 else 1


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
@pytest.mark.parametrize("i", range(len(PERMUTE_CASES)))
def test_permuted_view_made_contiguous(dt, i):
    shape, perm = PERMUTE_CASES[i]
    x = R.fill(shape, dt, 500 + i, F(dt))
    st = R.dense_strides(shape)
    got = R.oracle_repack(x, [shape[p] for p in perm], [st[p] for p in perm])
    want = GOLD[f"permute_{dt}_{i}"]
    assert got.shape == want.shape and got.tobytes() == want.tobytes()
    assert got.tobytes() == np.ascontiguousarray(x.transpose(perm)).tobytes()   # numpy agrees


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
@pytest.mark.parametrize("i", range(len(SLICE_CASES)))
def test_slice(dt, i):
    shape, b, e = SLICE_CASES[i]
    x = R.fill(shape, dt, 600 + i, F(dt))
    got = R.oracle_slice(x, b, e)
    want = GOLD[f"slice_{dt}_{i}"]
    assert got.shape == want.shape and got.tobytes() == want.tobytes()
    if pins_view_route(shape, b, e):
        # Tensor::slice keeps the strides and moves the offset; contiguous() gathers the window
        st = R.dense_strides(shape)
        off = sum(lo * s for lo, s in zip(b, st))
        view = R.oracle_repack(x, [hi - lo for lo, hi in zip(b, e)], st, off)
        assert view.tobytes() == GOLD[f"sliceview_{dt}_{i}"].tobytes()


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
@pytest.mark.parametrize("i", range(len(CONCAT_CASES)))
def test_concat(dt, i):
    shapes, dim = CONCAT_CASES[i]
    parts = [R.fill(sh, dt, 700 + 10 * i + j, F(dt)) for j, sh in enumerate(shapes)]
    got = R.oracle_concat(parts, dim)
    want = GOLD[f"concat_{dt}_{i}"]
    assert got.shape == want.shape and got.tobytes() == want.tobytes()


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
def test_transpose_2d(dt):
    x = R.fill((37, 66), dt, 800, F(dt))
    assert R.oracle_transpose(x).tobytes() == GOLD[f"transpose_{dt}"].tobytes()


@pytest.mark.parametrize("i", range(len(MUL_VIEW_CASES)))
def test_product_of_views_is_product_of_their_contiguous_copies(i):
    """ops::Mul on permuted views made contiguous, as the reference computes it (CPU backend:
    half inputs give FLOAT32), against repack + matmul of the restatement."""
    dt, sa, pa, sb, pb = MUL_VIEW_CASES[i]
    a = R.fill(sa, dt, 900 + i, F(dt)); b = R.fill(sb, dt, 950 + i, F(dt))
    sta, stb = R.dense_strides(sa), R.dense_strides(sb)
    av = R.oracle_repack(a, [sa[p] for p in pa], [sta[p] for p in pa])
    bv = R.oracle_repack(b, [sb[p] for p in pb], [stb[p] for p in pb])
    c, dtc = R.oracle_matmul(av, dt, bv, dt, "cpu")
    assert dtc == int(GOLD[f"mulview_{i}_dt"])
    assert c.tobytes() == GOLD[f"mulview_{i}"].tobytes()


@pytest.mark.skipif(not R.have_ref(), reason="reference library not built here")
def test_live_reference_larger_cases():
    x = R.fill((6, 130, 70), R.BFLOAT16, 1)
    st = R.dense_strides(x.shape)
    for perm in ((0, 2, 1), (1, 0, 2), (2, 1, 0)):
        got = R.oracle_repack(x, [x.shape[p] for p in perm], [st[p] for p in perm])
        assert got.tobytes() == R.ref_permute_contiguous(x, R.BFLOAT16, perm).tobytes()
    y = R.fill((300, 257), R.FLOAT32, 2)
    assert R.oracle_slice(y, [100, 0], [228, 257]).tobytes() == R.ref_slice(y, R.FLOAT32, [100, 0], [228, 257]).tobytes()
    parts = [R.fill((n, 129), R.INT8, 3 + n, 1) for n in (128, 1, 77)]
    assert R.oracle_concat(parts, 0).tobytes() == R.ref_concat(parts, R.INT8, 0).tobytes()


@pytest.mark.skipif(not R.have_ref(), reason="reference library not built here")
def test_reference_drops_the_offset_of_a_leading_slice_view():
    """Documents the one reference behaviour the restatement does not copy: contiguous() of a
    leading-dimension slice view returns the rows from 0 on (is_contiguous() passes and the copy
    ignores Metadata::offset, src/tensor.cpp:312-322, 396-403)."""
    y = R.fill((6, 7), R.INT16, 2, 1)
    v = R.ref_slice(y, R.INT16, [2], [5], view=True)
    assert np.array_equal(v, y[0:3]) and not np.array_equal(v, y[2:5])
    st = R.dense_strides(y.shape)
    assert np.array_equal(R.oracle_repack(y, (3, 7), st, 2 * 7), y[2:5])


def test_typecast_matches_the_reference_fixtures():
    """ops::Typecast: every cast the reference allows, bit for bit (float16 -> bfloat16 apart, see
    oracle/typecast_oracle.c), and the same refusals with the same messages."""
    casts = pinned_casts()
    assert len(casts) == 21
    for sdt, ddt in casts:
        got = R.oracle_typecast(typecast_input(sdt), sdt, ddt)
        assert got.tobytes() == GOLD[f"cast_{sdt}_{ddt}"].tobytes(), (R.DTYPE_NAMES[sdt], R.DTYPE_NAMES[ddt])
    rejected = {str(x).split(":", 1)[0]: str(x).split(":", 1)[1] for x in GOLD["cast_rejected"]}
    for sdt in range(8):
        for ddt in range(8):
            key = f"{sdt}>{ddt}"
            assert (key in rejected) == (not R.oracle_cast_valid(sdt, ddt)), key
            if key in rejected:
                assert rejected[key] == f"Invalid typecast from {R.DTYPE_NAMES[sdt]} to {R.DTYPE_NAMES[ddt]}"


def test_typecast_into_half_types_rounds_to_nearest_even():
    """The casts INTO float16 / bfloat16, checked against numpy (float16) and against the
    round-to-nearest-even bit arithmetic (bfloat16)."""
    x = typecast_input(R.FLOAT32)
    assert R.oracle_typecast(x, R.FLOAT32, R.FLOAT16).tobytes() == x.astype(np.float16).tobytes()
    h = typecast_input(R.FLOAT16)
    f = h.astype(np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    want = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    assert R.oracle_typecast(h, R.FLOAT16, R.BFLOAT16).tobytes() == want.tobytes()
    b = typecast_input(R.BFLOAT16)
    assert R.oracle_typecast(b, R.BFLOAT16, R.FLOAT16).tobytes() == R.bf16_bits_to_f32(b).astype(np.float16).tobytes()
