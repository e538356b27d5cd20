"""The arithmetic behind the integer-MMA INT8 decode kernel (csrc/bf16_decode_gemm.cu, I8 form), restated in
numpy: a bf16 token row x is written as X = rint(x * 2^(26 - e)) (e: |x| < 2^e for the whole row) in four
balanced base-128 digits; the kernel multiplies the digit planes with the int8 codes as integers and folds
the four int32 sums.  This file checks the claims the kernel's comments make about that representation; the
kernel itself is checked against the oracle on a GPU (tests/test_zm_gpu_w8_i8_decode.py)."""
import numpy as np


def _bf16_round(x):
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def _digits(x):
    amax = float(np.abs(x).max())
    e = int(np.floor(np.log2(amax))) + 1 if amax > 0 else 0
    X = np.rint(x.astype(np.float64) * 2.0 ** (26 - e)).astype(np.int64)
    planes, rest = [], X.copy()
    for _ in range(4):
        d = ((rest + 64) & 127) - 64
        rest = (rest - d) >> 7
        planes.append(d)
    return X, planes, rest, e


def test_digits_are_int8_and_reconstruct_the_integer():
    rng = np.random.default_rng(0)
    for scale in (1.0, 2.0 ** -20, 2.0 ** 15, 3.7):
        x = _bf16_round(rng.standard_normal(4096).astype(np.float32) * scale)
        x[7] = _bf16_round(np.float32(np.abs(x).max() * 0.999))  # an element next to the largest
        X, planes, rest, e = _digits(x)
        assert np.all(rest == 0)                      # four digits always suffice
        assert np.abs(X).max() <= 2 ** 26
        for d in planes:
            assert d.min() >= -64 and d.max() <= 63   # every digit is an int8 (with room to spare)
        back = sum(d * 128 ** i for i, d in enumerate(planes))
        assert np.array_equal(back, X)


def test_elements_within_2_to_minus_19_of_the_largest_are_exact():
    rng = np.random.default_rng(1)
    x = _bf16_round(rng.standard_normal(2048).astype(np.float32))
    x[::7] *= np.float32(2.0 ** -12)                   # a wide spread of magnitudes in one row
    x = _bf16_round(x)
    X, _, _, e = _digits(x)
    recon = X.astype(np.float64) * 2.0 ** (e - 26)
    big = np.abs(x) >= np.abs(x).max() * 2.0 ** -19
    assert np.array_equal(recon[big], x[big].astype(np.float64))
    assert np.abs(recon - x).max() <= 2.0 ** (e - 27)  # the rest: rounded to 2^-27 of the row's scale


def test_folded_integer_product_equals_the_product_of_the_reconstruction():
    rng = np.random.default_rng(2)
    x = _bf16_round(rng.standard_normal(1024).astype(np.float32))
    q = rng.integers(-127, 128, size=(16, 1024), dtype=np.int64)
    X, planes, _, e = _digits(x)
    sums = [q @ d for d in planes]                     # what the four column blocks of the MMA hold
    for s in sums:
        assert np.abs(s).max() < 2 ** 31                # int32 accumulators cannot overflow (|q d| <= 8128 per term)
    folded = ((sums[3] * 128 + sums[2]) * 128 + sums[1]) * 128 + sums[0]
    assert np.array_equal(folded, q @ X)
