"""Parity on the shapes that are benchmarked: the canonical 4096^3 problem in full, the prefill
projection shapes (M = 2048 with N or K = 11008), the decode pairs (M in {1, 16, 64}) and one shard of
the N-sharded 16384 x 28672 x 8192 problem under the default planner.

Every call goes through the C ABI.  Tolerances: conversions, O2 activation codes and scales and the O1
output bit-exact; O0/O2 outputs rtol = atol = 1e-3 (the reference's own GPU tests,
tests/integration/test_sm120_o{0,1,2}.py); MSE of O1/O2 against O0 within 2 % of the oracle's.
Inputs come from the CUDA quantizers (bit-identical to the oracle's, see test_gpu_prepare.py) so that
the large cases do not spend their time in the CPU generator.
"""

import numpy as np
import pytest

from oracle import adangel_oracle as orc

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-3


@pytest.fixture(scope="module")
def K():
    from adangel_oyzl_b200 import kernels

    return kernels


def _inputs(m, n, k, seed):
    from adangel_oyzl_b200 import synthetic

    return synthetic.canonical_inputs(m, n, k, seed=seed, device="cuda")


def _run_all(K, p, variants=("o0", "o1", "o2")):
    out = {}
    if "o0" in variants:
        out["a16"], out["w16"] = K.int8_to_fp16(p.A_int8, p.A_scale), K.mxfp4_to_fp16(p.W_mxfp4, p.W_scale)
        out["o0"] = K.gemm_o0(out["a16"], out["w16"])
    if "o1" in variants:
        out["w8"] = K.mxfp4_to_int8(p.W_mxfp4)
        out["o1"] = K.gemm_o1(p.A_int8, p.A_scale, out["w8"], p.W_scale)
        if p.A_int8.shape[0] > 64:
            weights = K.O1Weights(p.W_mxfp4, p.W_scale)
            out["o1_linear"] = K.o1_linear(p.A_int8, p.A_scale, weights)
    if "o2" in variants:
        out["codes"], out["sf"], sfa = K.o2_quantize_activation(p.A_int8, p.A_scale)
        out["o2"] = K.gemm_o2(out["codes"], sfa, p.W_mxfp4, K.o2_tile_scales(p.W_scale))
    K.check_status()
    return out


def _host(p, rows=None):
    sel = slice(None) if rows is None else rows
    return (p.A_int8[sel].cpu().numpy(), p.A_scale[sel].cpu().numpy(), p.W_mxfp4.cpu().numpy(), p.W_scale.cpu().numpy())


def _check_rows(got, host, rows=None, variants=("o0", "o1", "o2")):
    """Compare the GPU results on `rows` (all rows if None) with the oracle; returns the oracle outputs."""
    sel = slice(None) if rows is None else rows.cpu().numpy()
    want = {}
    if "o0" in variants:
        want["o0"] = orc.run_o0(*host)["output"]
        np.testing.assert_allclose(got["o0"].cpu().numpy()[sel], want["o0"], rtol=RTOL, atol=ATOL)
    if "o1" in variants:
        want["o1"] = orc.run_o1(*host)["output"]
        np.testing.assert_array_equal(got["o1"].cpu().numpy()[sel], want["o1"])
        if "o1_linear" in got:
            np.testing.assert_array_equal(got["o1_linear"].cpu().numpy()[sel], want["o1"])
    if "o2" in variants:
        r2 = orc.run_o2(*host)
        want["o2"] = r2["output"]
        np.testing.assert_array_equal(got["codes"].cpu().numpy()[sel], r2["converted_activation"][0])
        np.testing.assert_array_equal(got["sf"].cpu().numpy()[sel], r2["converted_activation"][1])
        np.testing.assert_allclose(got["o2"].cpu().numpy()[sel], want["o2"], rtol=RTOL, atol=ATOL)
    return want


def test_canonical_4096_every_row(K):
    """All 4096 rows of the canonical problem: conversions, codes, scales and O1 bit-exact, O0/O2 within
    1e-3, and the MSE of O1 and O2 against O0 within 2 % of the oracle's."""
    p = _inputs(4096, 4096, 4096, seed=20250805)
    got = _run_all(K, p)
    host = _host(p)
    np.testing.assert_array_equal(got["w16"].cpu().numpy().view(np.uint16),
                                  orc.dequantize_mxfp4(host[2], host[3], np.float16).view(np.uint16))
    np.testing.assert_array_equal(got["a16"].cpu().numpy().view(np.uint16),
                                  orc.dequantize_int8_per_row(host[0], host[1], np.float16).view(np.uint16))
    np.testing.assert_array_equal(got["w8"].cpu().numpy(), orc.mxfp4_to_int8_base(host[2]))
    want = _check_rows(got, host)
    y0, y1, y2 = (got[v].cpu().numpy() for v in ("o0", "o1", "o2"))
    assert orc.mse_fp64(y1, y0) == pytest.approx(orc.mse_fp64(want["o1"], want["o0"]), rel=0.02)
    assert orc.mse_fp64(y2, y0) == pytest.approx(orc.mse_fp64(want["o2"], want["o0"]), rel=0.02)


@pytest.mark.parametrize("shape", [(2048, 4096, 4096), (2048, 11008, 4096), (2048, 4096, 11008)])
def test_prefill_projection_shapes(K, shape):
    """M = 2048 projections: N = 11008 ends in a partial 256-wide tile, K = 11008 is 344 K32 groups (43 O2 K
    slabs).  256 rows spread over every 128-row block against the oracle, all columns."""
    import torch

    m, n, k = shape
    p = _inputs(m, n, k, seed=20250805 + 3)
    got = _run_all(K, p)
    rows = torch.arange(3, m, 8, device="cuda")
    want = _check_rows(got, _host(p, rows), rows)
    sel = rows.cpu().numpy()
    y0 = got["o0"].cpu().numpy()[sel]
    assert orc.mse_fp64(got["o1"].cpu().numpy()[sel], y0) == pytest.approx(orc.mse_fp64(want["o1"], want["o0"]), rel=0.02)
    assert orc.mse_fp64(got["o2"].cpu().numpy()[sel], y0) == pytest.approx(orc.mse_fp64(want["o2"], want["o0"]), rel=0.02)
    for v in ("o0", "o1", "o2"):
        assert bool(torch.isfinite(got[v]).all())


@pytest.mark.parametrize("nk", [(4096, 4096), (11008, 4096)])
@pytest.mark.parametrize("m", [1, 16, 64])
def test_decode_pairs(K, m, nk):
    """The decode pairs, O1 and O2, every element."""
    n, k = nk
    p = _inputs(m, n, k, seed=20250805 + 4)
    got = _run_all(K, p, variants=("o1", "o2"))
    _check_rows(got, _host(p), variants=("o1", "o2"))


def test_sharded_shape_shard_default_planner(K, monkeypatch):
    """One shard of the 16384 x 28672 x 8192 problem split eight ways (N = 3584) with the planner left to
    itself: O2 and O0 must pick the CTA-pair kernels here, and their results must match the oracle on 64 rows
    spread over all row blocks (every column)."""
    import torch

    from adangel_oyzl_b200.ops import _sm100

    monkeypatch.delenv("ADG_TWO_CTA", raising=False)
    m, n, k = 16384, 3584, 8192
    assert _sm100.plan_info("o2", m, n, k)["kernel_symbol"].startswith("gemm_pair_kernel<2")
    assert _sm100.plan_info("o0", m, n, k)["kernel_symbol"].startswith("gemm_pair_kernel<0")
    p = _inputs(m, n, k, seed=20250805 + 5)
    got = _run_all(K, p)
    rows = torch.arange(77, m, 256, device="cuda")
    assert rows.numel() == 64
    _check_rows(got, _host(p, rows), rows)
    for v in ("o0", "o1", "o2"):
        assert bool(torch.isfinite(got[v]).all())
