"""The arithmetic behind the W8A32 integer tensor-core route, restated in numpy (no GPU): fp32 activations scaled per
row by a power of two into [2^29, 2^30), rounded to int32 and cut into four signed base-256 digits; the four int8 x int8
dot products recombined in 64-bit integers.  Checks that the digits are int8, that they reproduce the integer, and
that the result stays within 1e-7 of the float64 value of the reference's sum (src/core/quantize.c:100-177) — also
with an outlier 1000x the other activations, the case a coarser grid would fail."""
import numpy as np
import pytest


def digit_planes(a):
    mx = np.abs(a).max(axis=1)
    e = np.floor(np.log2(np.where(mx > 0, mx, 1.0))).astype(np.int64)
    sexp = np.where(mx > 0, np.minimum(29 - e, 126), 0)
    v = np.rint(a.astype(np.float64) * np.ldexp(1.0, sexp)[:, None]).astype(np.int64)
    digits, t = [], v.copy()
    for _ in range(4):
        d = ((t & 0xFF) ^ 0x80) - 0x80          # signed low byte
        t = (t - d) >> 8
        digits.append(d)
    assert np.all(t == 0)
    return v, digits, sexp


@pytest.mark.parametrize("outlier", [False, True])
def test_digits_are_int8_and_exact(outlier):
    rng = np.random.default_rng(5)
    M, N, K = 6, 96, 4096
    a = rng.standard_normal((M, K)).astype(np.float32)
    if outlier:
        a[0, 7] = 1000.0
    q = rng.integers(-127, 128, (N, K)).astype(np.int64)
    v, digits, sexp = digit_planes(a)
    assert all(d.min() >= -128 and d.max() <= 127 for d in digits)
    assert np.array_equal(sum(d << (8 * j) for j, d in enumerate(digits)), v)
    assert np.abs(v).max() < 2 ** 30 + 1
    parts = [d @ q.T for d in digits]
    assert all(np.abs(p).max() < 2 ** 31 for p in parts)          # each fits the s32 accumulator
    total = sum(p << (8 * j) for j, p in enumerate(parts))
    got = total.astype(np.float64) * np.ldexp(1.0, -sexp)[:, None]
    want = a.astype(np.float64) @ q.T.astype(np.float64)
    assert np.abs(got - want).max() / np.abs(want).max() <= 1e-7
