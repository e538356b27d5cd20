"""Oracle of the dense W8A16 quantiser ([K, N] weights, one scale per (row group, column)) pinned to
the known-answer tests of the reference (src/tensor/quantizer.rs:969-1300, read as text)."""
import numpy as np

from oracle import oracle as orc


def _dequant(q, s, g):
    K = q.shape[0]
    g = g if g > 0 else K
    return q.astype(np.float32) * np.repeat(s, g, axis=0)[:K]


def test_int_multiples_of_the_scale_round_trip_exactly():
    # round_trip_bit_exact_for_int_multiples_of_scale: K=4, N=1, scale 1.0
    w = np.array([[2.0], [-4.0], [6.0], [-127.0]], dtype=np.float32)
    q, s = orc.absmax_per_group_symmetric(w)
    assert s.shape == (1, 1) and abs(float(s[0, 0]) - 1.0) < 1e-9
    np.testing.assert_array_equal(q.ravel(), [2, -4, 6, -127])
    np.testing.assert_array_equal(_dequant(q, s, 0), w)


def test_round_trip_error_within_one_over_127_for_unit_columns():
    k, n = 8, 3
    w = np.zeros((k, n), dtype=np.float32)
    for row in range(k):
        w[row, 0] = np.float32(-1.0) + np.float32(2.0) * np.float32(row) / np.float32(k - 1)
        w[row, 1] = 0.7 if row % 2 == 0 else -0.3
        w[row, 2] = -1.0 if row == 3 else 0.0
    q, s = orc.absmax_per_group_symmetric(w)
    assert q.shape == (k, n) and s.shape == (1, n)
    assert np.abs(w - _dequant(q, s, 0)).max() < 1.0 / 127.0 + 1e-6


def test_scales_length_contracts():
    assert orc.absmax_per_group_symmetric(np.full((5, 7), 0.5, np.float32))[1].shape == (1, 7)
    assert orc.absmax_per_group_symmetric(np.full((11, 13), 0.25, np.float32))[1].shape == (1, 13)
    assert orc.absmax_per_group_symmetric(np.full((256, 7), 0.5, np.float32), 128)[1].size == 14
    assert orc.absmax_per_group_symmetric(np.full((200, 7), 0.5, np.float32), 128)[1].size == 14
    assert orc.absmax_per_group_symmetric(np.full((5, 7), 0.5, np.float32), 5)[1].size == 7


def test_all_zero_column_gets_the_floor_scale():
    q, s = orc.absmax_per_group_symmetric(np.zeros((4, 2), np.float32))
    assert (s >= np.float32(1e-12)).all() and (s == np.float32(1e-12)).all()
    assert (q == 0).all() and (_dequant(q, s, 0) == 0).all()


def test_outlier_stays_inside_its_group():
    k, g = 256, 128
    w = np.zeros((k, 1), dtype=np.float32)
    w[:128, 0] = np.where(np.arange(128) % 2 == 0, 0.001, -0.001)
    w[200, 0] = 100.0
    q, s = orc.absmax_per_group_symmetric(w, g)
    assert s.size == 2
    err_pg = np.abs(w - _dequant(q, s, g))[:128].max()
    assert err_pg < 1e-4
    qc, sc = orc.absmax_per_group_symmetric(w)
    assert sc.size == 1
    err_pc = np.abs(w - _dequant(qc, sc, 0))[:128].max()
    assert err_pc > err_pg * 50.0


def test_ramp_round_trip_per_group():
    k, n, g = 256, 3, 128
    w = np.repeat((np.float32(-1.0) + np.float32(2.0) * np.arange(k, dtype=np.float32) / np.float32(k - 1))[:, None], n, 1)
    q, s = orc.absmax_per_group_symmetric(w.astype(np.float32), g)
    assert np.abs(w - _dequant(q, s, g)).max() < 1.0 / 127.0 + 1e-6


def test_full_column_group_equals_per_channel():
    k, n = 8, 3
    w = (np.arange(k * n, dtype=np.float32) * np.float32(0.1) - np.float32(0.4)).reshape(k, n)
    qc, sc = orc.absmax_per_group_symmetric(w)
    qg, sg = orc.absmax_per_group_symmetric(w, k)
    np.testing.assert_array_equal(qc, qg)
    np.testing.assert_array_equal(sc, sg)


def test_against_numpy_restatement_and_special_values():
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((77, 19)) * 0.02).astype(np.float32)
    w[3, 4] = np.nan
    w[10, 7] = np.inf
    w[11, 7] = 1.0
    g = 32
    q, s = orc.absmax_per_group_symmetric(w, g)
    for gi in range(3):
        blk = w[gi * g:(gi + 1) * g]
        amax = np.where(np.isnan(blk), 0, np.abs(blk)).max(axis=0).astype(np.float32)
        np.testing.assert_array_equal(s[gi], np.maximum(amax / np.float32(127.0), np.float32(1e-12)))
    assert q[3, 4] == 0            # NaN quotient -> 0
    assert q[10, 7] == 0           # inf / inf = NaN -> 0
    assert q[11, 7] == 0           # finite / inf = 0
    with np.errstate(invalid="ignore", divide="ignore"):
        quo = w / np.repeat(s, g, axis=0)[:77]
    exp = np.where(np.isnan(quo), 0, np.clip(np.sign(quo) * np.floor(np.abs(quo) + np.float32(0.5)), -127, 127))
    np.testing.assert_array_equal(q, exp.astype(np.int8))


def test_truncating_dequant_bits():
    rng = np.random.default_rng(6)
    q = rng.integers(-127, 128, size=(40, 24), dtype=np.int8)
    s = (rng.random((2, 24), dtype=np.float32) * 0.01 + 1e-4).astype(np.float32)
    got = orc.int8_to_bf16_per_group(q, s, 20)
    f = q.astype(np.float32) * np.repeat(s, 20, axis=0)
    np.testing.assert_array_equal(got, (f.view(np.uint32) >> 16).astype(np.uint16))
    # per channel
    got = orc.int8_to_bf16_per_group(q, s[:1])
    f = q.astype(np.float32) * s[:1]
    np.testing.assert_array_equal(got, (f.view(np.uint32) >> 16).astype(np.uint16))
