"""o1x, the exact-integer variant of O1 (an addition of this build, requested by name only).

Its arithmetic is deterministic (exact INT32 sum, one INT32 -> FP32 conversion, two FP32 multiplies), so the
GPU result is compared with the oracle's ``run_o1x`` bit for bit.  Against the literal O1 recurrence, which
rounds twice per K32 group, it agrees within rtol = 1e-4, atol = 1e-5 on the canonical distributions (the
literal path's accumulated rounding); column blocks that hold a W row whose scale codes spread over more than
3 take the literal kernel and must carry its bits.
"""

import numpy as np
import pytest

from oracle import adangel_oracle as orc
from tests.gpu_util import to_cuda

pytestmark = pytest.mark.gpu

RTOL_VS_LITERAL, ATOL_VS_LITERAL = 1e-4, 1e-5


@pytest.fixture(scope="module")
def K():
    from adangel_oyzl_b200 import kernels

    return kernels


def _run(K, a_int8, a_scale, w_mx, w_sc):
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    weights = K.O1xWeights(dw, dws)
    y = K.gemm_o1x(da, ds, weights)
    K.check_status()
    return y.cpu().numpy(), weights


@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 512, 1024), (1000, 768, 2048), (129, 1028, 448), (16, 256, 192),
                                   (1, 128, 64), (2048, 512, 11008)])
def test_o1x_matches_oracle_bit_for_bit(K, shape):
    m, n, k = shape
    args = orc.canonical_inputs(m, n, k, seed=59)
    want = orc.run_o1x(*args)
    got, weights = _run(K, *args)
    np.testing.assert_array_equal(weights.w_int8x.cpu().numpy(), want["converted_weight"])
    np.testing.assert_array_equal(weights.col_factor.cpu().numpy(), want["column_factor"])
    assert weights.ineligible_rows() == want["ineligible_rows"] == 0
    np.testing.assert_array_equal(got, want["output"])
    np.testing.assert_allclose(got, orc.run_o1(*args)["output"], rtol=RTOL_VS_LITERAL, atol=ATOL_VS_LITERAL)


def test_o1x_ineligible_rows_take_the_literal_kernel(K):
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(200, 640, 512, seed=61)
    w_sc = w_sc.copy()
    w_sc[3, 5] += 6        # spread 6+ in row 3     -> column block 0 literal
    w_sc[300, 1] = 90      # far below the others   -> column block 2 literal
    w_mx = w_mx.copy()
    w_mx[520, 16:32] = 0   # an all-zero block ...
    w_sc[520, 1] = 10      # ... whose odd scale code does not count: row 520 stays eligible
    want = orc.run_o1x(a_int8, a_scale, w_mx, w_sc)
    assert want["ineligible_rows"] == 2
    got, weights = _run(K, a_int8, a_scale, w_mx, w_sc)
    assert weights.ineligible_rows() == 2
    np.testing.assert_array_equal(weights.w_int8x.cpu().numpy(), want["converted_weight"])
    np.testing.assert_array_equal(got, want["output"])
    literal = orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"]
    np.testing.assert_array_equal(got[:, 0:128], literal[:, 0:128])
    np.testing.assert_array_equal(got[:, 256:384], literal[:, 256:384])
    np.testing.assert_allclose(got, literal, rtol=RTOL_VS_LITERAL, atol=ATOL_VS_LITERAL)


def test_o1x_worst_case_magnitudes_stay_exact(K):
    # |A| = 127, |W'| = 96 everywhere with equal signs: the largest INT32 sum the variant can meet
    m, n, k = 128, 128, 4096
    a_int8 = np.full((m, k), 127, dtype=np.int8)
    a_scale = np.full((m,), 0.01, dtype=np.float32)
    w_mx = np.full((n, k // 2), 0x77, dtype=np.uint8)   # +6 everywhere -> base 12
    w_sc = np.full((n, k // 32), 120, dtype=np.uint8)
    w_sc[:, 0] = 117                                     # min code 117: every other block is shifted by 3
    want = orc.run_o1x(a_int8, a_scale, w_mx, w_sc)
    got, _ = _run(K, a_int8, a_scale, w_mx, w_sc)
    np.testing.assert_array_equal(got, want["output"])


@pytest.mark.parametrize("mode", ["conversion_only", "compute_only", "cold", "steady_state"])
def test_o1x_through_the_harness(K, mode):
    from adangel_oyzl_b200.ops import _sm100

    args = orc.canonical_inputs(256, 384, 512, seed=67)
    da, ds, dw, dws = to_cuda(*args)
    result = _sm100.benchmark("o1x", mode, da, ds, dw, dws, 1, 2, 2)
    want = {"conversion_only": {"weight_conversion", "total"}, "compute_only": {"gemm", "total"},
            "cold": {"weight_conversion", "gemm", "total"}, "steady_state": {"gemm", "total"}}[mode]
    assert set(result["timings_ms"]) == want
    assert result["o1x_ineligible_rows"] == 0
    assert "kind::i8" in result["kernel"]["mma_family"]
    np.testing.assert_array_equal(result["output"].cpu().numpy(), orc.run_o1x(*args)["output"])
