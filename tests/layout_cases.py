"""Cases of the layout operations (views made contiguous, slices, concatenation, views
multiplied) shared by the golden-vector generator and the tests, which regenerate the inputs
from the same seeds: permute case i uses seed 500+i, slice 600+i, concat part j of case i
700+10*i+j, transpose 800, multiplied views 900+i (A) and 950+i (B)."""
from refcheck import BFLOAT16, FLOAT16, FLOAT32, INT8, INT32, INT64

LAYOUT_DTYPES = [INT8, BFLOAT16, FLOAT32, INT64]           # 1-, 2-, 4- and 8-byte elements
PERMUTE_CASES = [((5, 7), (1, 0)), ((33, 65), (1, 0)), ((3, 4, 5), (0, 2, 1)), ((3, 4, 5), (1, 0, 2)),
                 ((3, 4, 5), (2, 0, 1)), ((2, 3, 4, 5), (3, 1, 0, 2)), ((4, 70, 40), (0, 2, 1))]
SLICE_CASES = [((6, 7), (1, 2), (5, 6)), ((10, 12), (0, 3), (10, 9)), ((4, 5, 6), (1, 0, 2), (3, 5, 5)),
               ((9, 8), (2, 0), (7, 8)), ((5, 6, 7), (0, 1, 0), (5, 4, 7))]
CONCAT_CASES = [([(2, 6), (3, 6), (1, 6)], 0), ([(4, 2), (4, 5)], 1), ([(2, 3, 4), (2, 5, 4), (2, 1, 4)], 1),
                ([(2, 3, 4), (2, 3, 2)], 2), ([(70, 33), (58, 33)], 0)]
MUL_VIEW_CASES = [  # (dtype, stored A shape, perm A, stored B shape, perm B)
    (FLOAT32, (9, 12), (1, 0), (9, 7), (0, 1)), (FLOAT32, (12, 9), (0, 1), (7, 9), (1, 0)),
    (INT8, (9, 12), (1, 0), (7, 9), (1, 0)), (BFLOAT16, (2, 9, 12), (0, 2, 1), (2, 7, 9), (0, 2, 1)),
    (FLOAT16, (12, 2, 9), (1, 0, 2), (2, 9, 7), (0, 1, 2)), (INT32, (6, 5), (1, 0), (4, 6), (1, 0))]


def pins_view_route(shape, begin, end) -> bool:
    """Tensor::slice(...).contiguous() is pinned only where the view is not a leading-dimension
    slice: there the reference drops the view's offset (see oracle/layout_oracle.c)."""
    return any(lo != 0 or hi != n for lo, hi, n in list(zip(begin, end, shape))[1:])


def typecast_input(sdt: int, n: int = 4099):
    """Seeded source values for the typecast cases: integers in [-10, 10]; floats spread over
    [-300, 300) so that float -> integer truncation and half rounding are exercised."""
    import numpy as np
    import refcheck as R
    if sdt <= INT64:
        return R.fill((n,), sdt, 970 + sdt, 1)
    x = R.to_f64(R.fill((n,), FLOAT32, 970 + sdt), FLOAT32) * 300.0
    if sdt == FLOAT32:
        return x.astype(np.float32)
    if sdt == FLOAT16:
        return x.astype(np.float16)
    if sdt == BFLOAT16:
        return R.f32_to_bf16_bits(x.astype(np.float32))
    return x + 1e-9 * x   # float64: values that are not exactly representable in float32


# the casts whose reference HOST arithmetic is sound (everything but float16 -> bfloat16, where the
# reference's bfloat16_t(float) constructor zeroes normal values)
def pinned_casts():
    import refcheck as R
    return [(s, d) for s in range(8) for d in range(8)
            if s != d and R.oracle_cast_valid(s, d) and not (s == FLOAT16 and d == BFLOAT16)]
