"""CPU checks of the oracle's statement of o1x, the exact-integer O1 variant of this build (the reference
has no such variant; its O1 is the per-K32 recurrence, python/adangel/reference/o1.py:8-29).  The shifted INT8
image must reproduce the per-group partials exactly, and the result must stay within the stated tolerance of
the literal recurrence: rtol = 1e-4, atol = 1e-5."""

import numpy as np

from oracle import adangel_oracle as orc


def test_shifted_image_reproduces_scaled_partials_exactly():
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(32, 96, 512, seed=5)
    w_shift, factor, eligible = orc.o1x_prepare(w_mx, w_sc)
    assert eligible.all() and np.abs(w_shift.astype(np.int32)).max() <= 96
    partials = orc.o1_partials(a_int8, orc.mxfp4_to_int8_base(w_mx)).astype(np.float64)  # [m, n, g]
    scaled = (partials * np.ldexp(1.0, w_sc.astype(np.int64) - 128)[None, :, :]).sum(axis=2)  # exact in FP64
    sums = a_int8.astype(np.int64) @ w_shift.astype(np.int64).T
    np.testing.assert_array_equal(sums.astype(np.float64) * factor.astype(np.float64)[None, :], scaled)


def test_o1x_tracks_literal_o1_within_stated_tolerance():
    args = orc.canonical_inputs(64, 256, 4096, seed=9)
    got = orc.run_o1x(*args)
    assert got["ineligible_rows"] == 0
    np.testing.assert_allclose(got["output"], orc.run_o1(*args)["output"], rtol=1e-4, atol=1e-5)


def test_wide_spread_rows_fall_back_in_blocks_of_128_columns():
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(16, 384, 256, seed=11)
    w_sc = w_sc.copy()
    w_sc[130, 2] += 5
    got = orc.run_o1x(a_int8, a_scale, w_mx, w_sc)
    literal = orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"]
    assert got["ineligible_rows"] == 1
    np.testing.assert_array_equal(got["output"][:, 128:256], literal[:, 128:256])
    assert (got["converted_weight"][130] == 0).all() and got["column_factor"][130] == 0.0
    w_mx = w_mx.copy()
    w_mx[130, 32:48] = 0  # the odd block holds only zeros now: it no longer counts
    assert orc.run_o1x(a_int8, a_scale, w_mx, w_sc)["ineligible_rows"] == 0
