"""Generates the golden fixtures in this folder from the REFERENCE LIBRARY ITSELF.

    make -C oracle ref          # builds oracle/_ref/libtv_ref_cpu.so from the reference tree
    python tests/golden/make_golden.py

The reference's own tests hold no expected values for matmul (tests/mul.cpp only times),
so the pin is the reference's implementation run here on seeded inputs:

  golden_small.npz    every (A dtype, B dtype) pair, one 2-D and one batched 3-D case on the
                      small-output path (mul_kernel_basic, src/backend/cpu/mul.cpp:7-25)
  golden_tiled.npz    the large-output path (mul_kernel_tiled<64>, mul.cpp:27-85): sampled rows
                      and a SHA-256 of the whole result
  golden_configs.npz  sampled rows of the five benchmark configurations at FULL size
  golden_layout.npz   the layout operations either side of the matmul: permute().contiguous(),
                      ops::Slice, slice().contiguous(), ops::Concat, ops::Transpose, ops::Mul of
                      permuted views made contiguous, and ops::Typecast (the casts it allows, its
                      refusals with their messages)
  golden_meta.json    compute_type table, the messages ops::Mul throws for bad shapes
                      (src/ops.cpp:540-556), thread count, sizes

Inputs are not stored: they are regenerated from their seeds (tests/refcheck.py `fill`), and
their SHA-256 is stored so that a drifting generator is caught.

Rows of a tiled result depend only on the same rows of A (and all of B), so for the big
configurations the reference is run on a subset of A's rows that still takes the tiled path
(>= 1 Mi outputs); configuration 1 is also run in full to check that claim bit for bit.
"""
from __future__ import annotations

import json
import sys
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import refcheck as R  # noqa: E402

F = lambda dt: 0 if dt >= R.BFLOAT16 else 1  # dist: floats uniform [-1,1), ints [-10,10]


def small():
    out = {}
    for a in range(8):
        for b in range(8):
            A = R.fill((5, 7), a, 1000 + a, F(a)); B = R.fill((7, 6), b, 2000 + b, F(b))
            c, dt = R.ref_matmul(A, a, B, b)
            out[f"m2_{a}_{b}"] = c
            out[f"m2_{a}_{b}_dt"] = np.int32(dt)
            A = R.fill((2, 3, 4), a, 3000 + a, F(a)); B = R.fill((2, 4, 5), b, 4000 + b, F(b))
            c, dt = R.ref_matmul(A, a, B, b)
            out[f"m3_{a}_{b}"] = c
            out[f"m3_{a}_{b}_dt"] = np.int32(dt)
    np.savez_compressed(HERE / "golden_small.npz", **out)


TILED_CASES = [  # (name, dtype a, dtype b, shape a, shape b)
    ("f32", 6, 6, (1024, 200), (200, 1024)),
    ("i8", 0, 0, (1024, 200), (200, 1024)),
    ("bf16", 4, 4, (1024, 200), (200, 1024)),
    ("f16", 5, 5, (1024, 200), (200, 1024)),
    ("i32", 2, 2, (1024, 200), (200, 1024)),
    ("f64", 7, 7, (1024, 200), (200, 1024)),
    ("i16_i8", 1, 0, (1024, 200), (200, 1024)),
    ("f32_i8", 6, 0, (1024, 200), (200, 1024)),
    ("i8_f32", 0, 6, (1024, 200), (200, 1024)),   # lossy on the CPU tiled path (A's type accumulates)
    ("f32_b3", 6, 6, (4, 520, 70), (4, 70, 520)),
    ("bf16_b3", 4, 4, (4, 520, 70), (4, 70, 520)),
    ("i8_b3", 0, 0, (4, 520, 70), (4, 70, 520)),
]
TILED_ROWS = [0, 1, 63, 64, 511, 1023]


def tiled():
    out, meta = {}, {}
    for name, a, b, sa, sb in TILED_CASES:
        A = R.fill(sa, a, 5000 + a, F(a)); B = R.fill(sb, b, 6000 + b, F(b))
        c, dt = R.ref_matmul(A, a, B, b)
        flat = c.reshape(-1, c.shape[-1])
        rows = [r for r in TILED_ROWS if r < flat.shape[0]] + [flat.shape[0] - 1]
        out[f"{name}_rows"] = flat[rows]
        meta[name] = {"dta": a, "dtb": b, "shape_a": sa, "shape_b": sb, "dtc": int(dt), "rows": rows,
                      "sha_a": R.sha(A), "sha_b": R.sha(B), "sha_c": R.sha(c)}
    np.savez_compressed(HERE / "golden_tiled.npz", **out)
    return meta


# the five benchmark configurations: (dtype, batch or None, M, K, N, dist)
CONFIGS = {
    1: (R.FLOAT32, None, 2592, 2048, 4096, 0),
    2: (R.BFLOAT16, None, 4096, 4096, 4096, 0),
    3: (R.FLOAT16, 32, 1024, 4096, 1024, 0),
    4: (R.INT8, None, 8192, 8192, 8192, 1),
    5: (R.FLOAT32, None, 65536, 4096, 4096, 0),
}
ROW_BLOCKS = 4       # four runs of 64 consecutive rows per configuration -> 256 rows through the reference
KEEP_PER_BLOCK = 4   # of which 4 per run are stored


def config_rows(cfg: int):
    """(batch index, row) pairs whose A rows go through the reference; deterministic."""
    dt, batch, M, K, N, _ = CONFIGS[cfg]
    if batch is None:
        starts = [0, (M // 3) // 64 * 64, (2 * M // 3) // 64 * 64 + 1, M - 64]
        return [(0, s + i) for s in starts for i in range(64)]
    # batched: 3 batches x 352 rows keeps the output above 1 Mi elements (tiled path)
    bs = [0, batch // 2 - 3, batch - 1]
    rows = list(range(0, 176)) + list(range(M - 176, M))
    return [(b, r) for b in bs for r in rows]


def kept_rows(cfg: int):
    dt, batch, M, K, N, _ = CONFIGS[cfg]
    pairs = config_rows(cfg)
    if batch is None:
        idx = [blk * 64 + j for blk in range(ROW_BLOCKS) for j in (0, 21, 42, 63)]
    else:
        per = len(pairs) // 3
        idx = [b * per + j for b in range(3) for j in (0, 100, 175, 176, 351)]
    return idx, [pairs[i] for i in idx]


def gen_rows(dt, ncols, pairs, rows_per_batch, seed, dist):
    """Rows (b, r) of a seeded [batch, rows, ncols] tensor, generated without the rest."""
    out = np.empty((len(pairs), ncols), dtype=R.NP[dt])
    for i, (b, r) in enumerate(pairs):
        out[i] = R.fill((ncols,), dt, seed, dist, first=(b * rows_per_batch + r) * ncols)
    return out


def configs():
    out, meta = {}, {}
    for cfg, (dt, batch, M, K, N, dist) in CONFIGS.items():
        t0 = time.time()
        seed_a, seed_b = R.SEED_BASE + 2 * cfg, R.SEED_BASE + 2 * cfg + 1
        pairs = config_rows(cfg)
        Asub = gen_rows(dt, K, pairs, M, seed_a, dist)
        if batch is None:
            B = R.fill((K, N), dt, seed_b, dist)
            c, dtc = R.ref_matmul(Asub, dt, B, dt)
        else:
            bs = sorted({b for b, _ in pairs})
            per = len(pairs) // len(bs)
            A3 = Asub.reshape(len(bs), per, K)
            B3 = np.stack([R.fill((K, N), dt, seed_b, dist, first=b * K * N) for b in bs])
            c, dtc = R.ref_matmul(A3, dt, B3, dt)
            c = c.reshape(-1, N)
        assert c.shape[0] * c.shape[1] >= 1024 * 1024, "must stay on the tiled path"
        idx, kept = kept_rows(cfg)
        out[f"c{cfg}_rows"] = c[idx]
        meta[str(cfg)] = {"dtype": dt, "batch": batch, "M": M, "K": K, "N": N, "dist": dist, "dtc_cpu": int(dtc),
                          "seed_a": seed_a, "seed_b": seed_b, "kept": kept, "sha_rows": R.sha(c[idx]),
                          "sha_a_rows": R.sha(Asub[idx])}
        if cfg == 1:  # the whole problem, to verify "a row of C depends on its row of A only"
            Afull = R.fill((M, K), dt, seed_a, dist)
            cfull, _ = R.ref_matmul(Afull, dt, B, dt)
            rows = [r for _, r in pairs]
            assert cfull[rows].tobytes() == c.tobytes(), "row-subset run differs from the full run"
            meta[str(cfg)]["sha_full"] = R.sha(cfull)
        print(f"config {cfg}: {time.time() - t0:.1f} s", flush=True)
    np.savez_compressed(HERE / "golden_configs.npz", **out)
    return meta


SHAPE_CASES = [((2, 3), (4, 5)), ((2, 3), (3,)), ((2, 3, 4), (3, 4, 5)), ((2, 3, 4), (2, 5, 5)), ((3,), (3,)),
               ((2, 3), (3, 4)), ((2, 3, 4, 5), (2, 3, 5, 4)), ((2, 3, 4), (2, 4, 6)), ((2, 3), (2, 3, 4))]


# ---- layout operations: views made contiguous, slices, concatenation, views multiplied ----------
from layout_cases import (CONCAT_CASES, LAYOUT_DTYPES, MUL_VIEW_CASES, PERMUTE_CASES, SLICE_CASES,  # noqa: E402
                          pinned_casts, pins_view_route, typecast_input)


def layout():
    out = {}
    for dt in LAYOUT_DTYPES:
        for i, (shape, perm) in enumerate(PERMUTE_CASES):
            out[f"permute_{dt}_{i}"] = R.ref_permute_contiguous(R.fill(shape, dt, 500 + i, F(dt)), dt, perm)
        for i, (shape, b, e) in enumerate(SLICE_CASES):
            x = R.fill(shape, dt, 600 + i, F(dt))
            out[f"slice_{dt}_{i}"] = R.ref_slice(x, dt, b, e)
            # the view route is pinned only where the view is not a leading-dimension slice:
            # there the reference drops the offset (see oracle/layout_oracle.c)
            if pins_view_route(shape, b, e):
                out[f"sliceview_{dt}_{i}"] = R.ref_slice(x, dt, b, e, view=True)
        for i, (shapes, dim) in enumerate(CONCAT_CASES):
            parts = [R.fill(sh, dt, 700 + 10 * i + j, F(dt)) for j, sh in enumerate(shapes)]
            out[f"concat_{dt}_{i}"] = R.ref_concat(parts, dt, dim)
        out[f"transpose_{dt}"] = R.ref_transpose2d(R.fill((37, 66), dt, 800, F(dt)), dt)
    for i, (dt, sa, pa, sb, pb) in enumerate(MUL_VIEW_CASES):
        c, dtc = R.ref_mul_permuted(R.fill(sa, dt, 900 + i, F(dt)), dt, pa, R.fill(sb, dt, 950 + i, F(dt)), dt, pb)
        out[f"mulview_{i}"] = c
        out[f"mulview_{i}_dt"] = np.int32(dtc)
    for sdt, ddt in pinned_casts():
        out[f"cast_{sdt}_{ddt}"] = R.ref_typecast(typecast_input(sdt), sdt, ddt)
    rejected = []
    for sdt in range(8):
        for ddt in range(8):
            try:
                R.ref_typecast(typecast_input(sdt, 8), sdt, ddt)
            except RuntimeError as e:
                rejected.append(f"{sdt}>{ddt}:{e}")
    out["cast_rejected"] = np.array(rejected)
    np.savez_compressed(HERE / "golden_layout.npz", **out)


def main():
    assert R.have_ref(), "build the reference first: make -C oracle ref"
    if "--layout-only" in sys.argv:
        layout()
        print("golden_layout.npz written to", HERE)
        return
    small()
    layout()
    meta = {"tiled": tiled(), "configs": configs()}
    meta["compute_type"] = [[int(R.ref().tvref_compute_type(a, b)) for b in range(8)] for a in range(8)]
    meta["shape_messages"] = [{"a": list(sa), "b": list(sb), "message": R.ref_validate(sa, sb)} for sa, sb in SHAPE_CASES]
    meta["threads"] = int(R.ref().tvref_threads())
    (HERE / "golden_meta.json").write_text(json.dumps(meta, indent=1))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
