"""Parity of the layout operations (tvb_repack, tvb_slice, tvb_concat, tvb_transpose2d) with the
restatement of the reference's clone_as_contiguous / ops::Slice / ops::Concat / ops::Transpose
and with the golden fixtures the reference library itself produced.  Byte moves: bit-exact."""
import ctypes as C

import numpy as np
import pytest

import refcheck as R
from gpuutil import Dev
from layout_cases import CONCAT_CASES, LAYOUT_DTYPES, PERMUTE_CASES, SLICE_CASES, pinned_casts, typecast_input

pytestmark = pytest.mark.gpu
GOLD = np.load(R.GOLDEN_DIR / "golden_layout.npz")
F = lambda dt: 0 if dt >= R.BFLOAT16 else 1
GUARD = 256


@pytest.fixture(scope="module")
def dev(tv):
    d = Dev(tv)
    yield d
    d.free_all()


def i64(v):
    return (C.c_int64 * len(v))(*[int(x) for x in v])


class Out:
    """A destination buffer with guard bands on both sides."""

    def __init__(self, dev, shape, dtype):
        self.dev, self.shape, self.dtype = dev, tuple(shape), dtype
        self.nbytes = int(np.prod(shape)) * R.NP[dtype]().itemsize
        self.raw = dev.alloc(self.nbytes + 2 * GUARD)
        canary = np.full(self.nbytes + 2 * GUARD, 0xA5, dtype=np.uint8)
        dev.check(dev.lib.tvb_memcpy_h2d(dev.device, self.raw, canary.ctypes.data, canary.nbytes, None))
        dev.sync()
        self.ptr = self.raw + GUARD

    def read(self):
        self.dev.sync()
        whole = self.dev.download(self.raw, (self.nbytes + 2 * GUARD,), R.INT8).view(np.uint8)
        assert (whole[:GUARD] == 0xA5).all() and (whole[-GUARD:] == 0xA5).all(), "write outside dst"
        out = whole[GUARD:GUARD + self.nbytes].copy().view(R.NP[self.dtype]).reshape(self.shape)
        self.dev.free(self.raw)
        return out


def gpu_repack(dev, storage, dt, shape, strides, offset=0):
    p = dev.upload(storage)
    out = Out(dev, shape, dt)
    dev.check(dev.lib.tvb_repack(dev.device, p + offset * storage.itemsize, out.ptr, dt, len(shape), i64(shape),
                                 i64(strides), None))
    res = out.read()
    dev.free(p)
    return res


def gpu_slice(dev, x, dt, begin, end):
    p = dev.upload(x)
    shape = [e - b for b, e in zip(begin, end)] + list(x.shape[len(begin):])
    out = Out(dev, shape, dt)
    dev.check(dev.lib.tvb_slice(dev.device, p, out.ptr, dt, x.ndim, i64(x.shape), len(begin), i64(begin), i64(end), None))
    res = out.read()
    dev.free(p)
    return res


def gpu_concat(dev, parts, dt, dim):
    ptrs = [dev.upload(p) for p in parts]
    shape = list(parts[0].shape)
    sizes = [p.shape[dim] for p in parts]
    shape[dim] = sum(sizes)
    out = Out(dev, shape, dt)
    arr = (C.c_void_p * len(ptrs))(*ptrs)
    dev.check(dev.lib.tvb_concat(dev.device, len(ptrs), arr, out.ptr, dt, len(shape), i64(parts[0].shape), i64(sizes),
                                 dim, None))
    res = out.read()
    for p in ptrs:
        dev.free(p)
    return res


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
@pytest.mark.parametrize("i", range(len(PERMUTE_CASES)))
def test_permuted_views_match_the_reference_fixtures(dev, dt, i):
    shape, perm = PERMUTE_CASES[i]
    x = R.fill(shape, dt, 500 + i, F(dt))
    st = R.dense_strides(shape)
    got = gpu_repack(dev, x, dt, [shape[p] for p in perm], [st[p] for p in perm])
    assert got.tobytes() == GOLD[f"permute_{dt}_{i}"].tobytes()


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
@pytest.mark.parametrize("i", range(len(SLICE_CASES)))
def test_slices_match_the_reference_fixtures(dev, dt, i):
    shape, b, e = SLICE_CASES[i]
    x = R.fill(shape, dt, 600 + i, F(dt))
    assert gpu_slice(dev, x, dt, b, e).tobytes() == GOLD[f"slice_{dt}_{i}"].tobytes()
    # the same window as a view (Tensor::slice keeps strides, moves the offset) made contiguous
    st = R.dense_strides(shape)
    off = sum(lo * s for lo, s in zip(b, st))
    got = gpu_repack(dev, x, dt, [hi - lo for lo, hi in zip(b, e)], st, off)
    assert got.tobytes() == GOLD[f"slice_{dt}_{i}"].tobytes()


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
@pytest.mark.parametrize("i", range(len(CONCAT_CASES)))
def test_concat_matches_the_reference_fixtures(dev, dt, i):
    shapes, dim = CONCAT_CASES[i]
    parts = [R.fill(sh, dt, 700 + 10 * i + j, F(dt)) for j, sh in enumerate(shapes)]
    assert gpu_concat(dev, parts, dt, dim).tobytes() == GOLD[f"concat_{dt}_{i}"].tobytes()


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
def test_transpose_2d_matches_the_reference_fixture(dev, dt):
    x = R.fill((37, 66), dt, 800, F(dt))
    p = dev.upload(x)
    out = Out(dev, (66, 37), dt)
    dev.check(dev.lib.tvb_transpose2d(dev.device, p, out.ptr, dt, 37, 66, None))
    assert out.read().tobytes() == GOLD[f"transpose_{dt}"].tobytes()
    dev.free(p)


# Larger and ragged cases against the restatement: every copy kernel, every vector width.
BIG_VIEWS = [
    # (stored shape, view shape, view strides, offset)
    ((512, 384), (384, 512), (1, 384), 0),                       # t(), everything 16-byte aligned: vector transpose
    ((3, 256, 160), (3, 160, 256), (40960, 1, 160), 0),          # permute {0,2,1}, aligned
    ((200, 144), (144, 200), (1, 144), 0),                       # t(), ragged tiles of whole vectors / words
    ((1000, 777), (777, 1000), (1, 777), 0),                     # t(): tiled transpose, ragged tiles
    ((5, 300, 260), (5, 260, 300), (78000, 1, 260), 0),          # permute {0,2,1}
    ((300, 5, 260), (5, 300, 260), (260, 1300, 1), 0),           # permute {1,0,2}: rows stay contiguous
    ((64, 96, 7), (7, 64, 96), (1, 672, 7), 0),                  # permute {2,0,1}: transpose with 2 outer... merged plane
    ((400, 512), (300, 384), (512, 1), 16 * 512 + 64),           # aligned inner window: 16-byte vectors
    ((400, 513), (300, 383), (513, 1), 3 * 513 + 5),             # ragged window: narrow vectors
    ((40, 50, 60), (20, 25, 30), (6000, 120, 2), 7),             # no contiguous run: element copy
    ((6, 8, 10, 12), (12, 8, 6, 10), (1, 120, 960, 12), 0),      # 4-D permute {3,1,0,2}
]


@pytest.mark.parametrize("dt", LAYOUT_DTYPES)
@pytest.mark.parametrize("case", BIG_VIEWS)
def test_views_made_contiguous(dev, dt, case):
    stored, shape, strides, off = case
    x = R.fill(stored, dt, 77, F(dt))
    want = R.oracle_repack(x, shape, strides, off)
    assert gpu_repack(dev, x, dt, shape, strides, off).tobytes() == want.tobytes()


@pytest.mark.parametrize("dt", [R.BFLOAT16, R.FLOAT32])
def test_row_shards_round_trip(dev, dt):
    """Slice on the leading dimension then Concat along it restores the tensor: the scatter and
    gather steps of the row-sharded matmul, each part one contiguous copy."""
    x = R.fill((1000, 384), dt, 5, F(dt))
    cuts = [0, 256, 512, 768, 1000]
    parts = [gpu_slice(dev, x, dt, [lo], [hi]) for lo, hi in zip(cuts[:-1], cuts[1:])]
    for (lo, hi), p in zip(zip(cuts[:-1], cuts[1:]), parts):
        assert p.tobytes() == R.oracle_slice(x, [lo], [hi]).tobytes()
    before = dev.lib.tvb_kernel_launches()
    back = gpu_concat(dev, parts, dt, 0)
    assert dev.lib.tvb_kernel_launches() == before      # copies only, no kernel
    assert back.tobytes() == x.tobytes() == R.oracle_concat(parts, 0).tobytes()


def test_concat_inner_dimension_large(dev):
    parts = [R.fill((300, n, 24), R.INT8, 9 + n, 1) for n in (5, 128, 31)]
    assert gpu_concat(dev, parts, R.INT8, 1).tobytes() == R.oracle_concat(parts, 1).tobytes()
    parts = [R.fill((123, 50, n), R.FLOAT16, 19 + n) for n in (8, 3, 64)]
    assert gpu_concat(dev, parts, R.FLOAT16, 2).tobytes() == R.oracle_concat(parts, 2).tobytes()


def test_double_transpose_is_identity_at_size(dev):
    """A size-independent property at a size the CPU checker would take long for: 8192 x 6144."""
    lib = dev.lib
    rows, cols = 8192, 6144
    a = dev.fill((rows, cols), R.BFLOAT16, 123)
    b = dev.alloc(rows * cols * 2)
    c = dev.alloc(rows * cols * 2)
    dev.check(lib.tvb_transpose2d(dev.device, a, b, R.BFLOAT16, rows, cols, None))
    dev.check(lib.tvb_transpose2d(dev.device, b, c, R.BFLOAT16, cols, rows, None))
    x = dev.download(a, (rows, cols), R.BFLOAT16)
    t = dev.download(b, (cols, rows), R.BFLOAT16)
    z = dev.download(c, (rows, cols), R.BFLOAT16)
    assert x.tobytes() == z.tobytes()
    assert np.array_equal(t[:64], x[:, :64].T) and np.array_equal(t[-5:], x[:, -5:].T)
    for p in (a, b, c):
        dev.free(p)


def test_argument_checks(dev):
    lib = dev.lib
    p = dev.alloc(4096)
    try:
        assert lib.tvb_repack(0, p, p, R.FLOAT32, 2, i64([4, 4]), i64([4, -1]), None) == 1     # negative stride
        assert lib.tvb_repack(0, p, p, R.FLOAT32, 9, i64([1] * 9), i64([1] * 9), None) == 2    # too many dims
        assert lib.tvb_repack(0, p, p, 9, 1, i64([4]), i64([1]), None) == 3                    # dtype
        assert lib.tvb_slice(0, p, p, R.FLOAT32, 2, i64([4, 4]), 2, i64([0, 2]), i64([4, 5]), None) == 2
        assert lib.tvb_slice(0, p, p, R.FLOAT32, 2, i64([4, 4]), 1, i64([3]), i64([3]), None) == 2
        arr = (C.c_void_p * 1)(p)
        assert lib.tvb_concat(0, 1, arr, p, R.FLOAT32, 2, i64([4, 4]), i64([4]), 2, None) == 2
        assert lib.tvb_concat(0, 0, arr, p, R.FLOAT32, 2, i64([4, 4]), i64([4]), 0, None) == 1
    finally:
        dev.free(p)


def test_torch_facing_layout_operators(tv):
    """The Python mirrors of ops::Slice / Concat / Transpose and Tensor::contiguous on torch tensors."""
    torch = pytest.importorskip("torch")
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randint(-100, 100, (6, 40, 56), device="cuda", generator=g, dtype=torch.int32)
    for view in (x.permute(0, 2, 1), x.permute(2, 0, 1), x[:, 3:29, 8:40], x[1:4], x.transpose(0, 1)[5:20]):
        assert torch.equal(tv.contiguous(view), view.contiguous())
    h = x.to(torch.bfloat16)
    assert torch.equal(tv.Slice(h, [(1, 5), (0, 40), (16, 48)]), h[1:5, :, 16:48])
    assert torch.equal(tv.Slice(h, [(2, 4), (0, 40), (0, 56)]), h[2:4])
    assert torch.equal(tv.Concat([h[:2], h[2:3], h[3:]], 0), h)
    assert torch.equal(tv.Concat([h[:, :, :24], h[:, :, 24:]], 2), h)
    m = x[0].to(torch.int8)
    assert torch.equal(tv.Transpose(m), m.t().contiguous())
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="Slice ranges cannot be empty"):
        tv.Slice(h, [])
    with pytest.raises(RuntimeError, match="second must be less than 40"):
        tv.Slice(h, [(0, 1), (0, 41), (0, 1)])
    with pytest.raises(ValueError, match="same dtype"):
        tv.Concat([h, x], 0)
    with pytest.raises(RuntimeError, match="only support 2D"):
        tv.Transpose(h)


def gpu_typecast(dev, x, sdt, ddt, misalign=0):
    p = dev.upload(np.concatenate([np.zeros(misalign, dtype=x.dtype), x]) if misalign else x)
    out = Out(dev, x.shape, ddt)
    rc = dev.lib.tvb_typecast(dev.device, p + misalign * x.itemsize, out.ptr, sdt, ddt, x.size, None)
    dev.check(rc)
    res = out.read()
    dev.free(p)
    return res


def test_typecast_matches_the_reference_fixtures_and_the_restatement(dev):
    """Every cast ops::Typecast allows, bit for bit: against the reference's own outputs where its
    host arithmetic is sound, against the restatement of the CUDA backend's rounding for all."""
    for sdt, ddt in pinned_casts():
        x = typecast_input(sdt)
        got = gpu_typecast(dev, x, sdt, ddt)
        assert got.tobytes() == GOLD[f"cast_{sdt}_{ddt}"].tobytes(), (R.DTYPE_NAMES[sdt], R.DTYPE_NAMES[ddt])
    for sdt in range(8):
        for ddt in range(8):
            if not R.oracle_cast_valid(sdt, ddt):
                continue
            x = typecast_input(sdt, 1003)
            assert gpu_typecast(dev, x, sdt, ddt).tobytes() == R.oracle_typecast(x, sdt, ddt).tobytes()
            # a source that starts off the pack boundary takes the element-wise route
            assert gpu_typecast(dev, x, sdt, ddt, misalign=1).tobytes() == R.oracle_typecast(x, sdt, ddt).tobytes()


def test_typecast_refusals(dev):
    lib = dev.lib
    p = dev.alloc(4096)
    try:
        for sdt in range(8):
            for ddt in range(8):
                rc = lib.tvb_typecast(0, p, p + 2048, sdt, ddt, 16, None)
                if R.oracle_cast_valid(sdt, ddt):
                    assert rc == 0
                else:
                    assert rc == 3   # TVB_ERR_DTYPE
                    assert lib.tvb_last_error_string().decode() == \
                        f"Invalid typecast from {R.DTYPE_NAMES[sdt]} to {R.DTYPE_NAMES[ddt]}"
        dev.sync()
        assert lib.tvb_typecast(0, None, p, R.INT8, R.FLOAT32, 16, None) == 1
    finally:
        dev.free(p)


def test_typecast_then_matmul_equals_the_mixed_pair(dev):
    """int8 x float16 -> FLOAT32: casting both operands to float32 first (what the promotion means)
    and multiplying gives the mixed-pair operator's result."""
    a = R.fill((96, 64), R.INT8, 3, 1); b = R.fill((64, 80), R.FLOAT16, 4)
    mixed, dt = dev.matmul(a, R.INT8, b, R.FLOAT16)
    af = gpu_typecast(dev, a, R.INT8, R.FLOAT32); bf = gpu_typecast(dev, b, R.FLOAT16, R.FLOAT32)
    both, dt2 = dev.matmul(af, R.FLOAT32, bf, R.FLOAT32)
    assert dt == dt2 == R.FLOAT32
    assert R.rel_frobenius(mixed, both, R.FLOAT32) <= 1e-5
