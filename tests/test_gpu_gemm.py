"""Parity of the three GEMM variants with the CPU oracle, through the C ABI and the ops surface.

Tolerances: INT32 K32 partials exact; O1 output bit-identical to the oracle (same operation order);
O0/O2 outputs within rtol = atol = 1e-3 (the tolerance of the reference's own GPU tests,
tests/integration/test_sm120_o{0,1,2}.py); MSE vs O0 within 2 % of the oracle's.
"""

import numpy as np
import pytest

from oracle import adangel_oracle as orc
from tests.gpu_util import golden_inputs, to_cuda

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-3
GOLDEN = ["canonical_128x128x128", "canonical_68x36x64", "fp16_seed2026_128x128x256", "fp16_seed2026_132x132x256",
          "edge_zero_128x128x256", "edge_alternating_128x128x256", "edge_saturated_128x128x256", "seed7_16x8x64"]


@pytest.fixture(scope="module")
def K():
    from adangel_oyzl_b200 import kernels

    return kernels


def _gpu_all(K, a_int8, a_scale, w_mx, w_sc, dump=False):
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    y0 = K.gemm_o0(K.int8_to_fp16(da, ds), K.mxfp4_to_fp16(dw, dws))
    r1 = K.gemm_o1(da, ds, K.mxfp4_to_int8(dw), dws, dump_partials=dump)
    codes, _, sfa = K.o2_quantize_activation(da, ds)
    y2 = K.gemm_o2(codes, sfa, dw, K.o2_tile_scales(dws))
    K.check_status()
    y1, partials = r1 if dump else (r1, None)
    return y0.cpu().numpy(), y1.cpu().numpy(), y2.cpu().numpy(), (partials.cpu().numpy() if dump else None)


def _compare(K, a_int8, a_scale, w_mx, w_sc, dump=True):
    y0, y1, y2, partials = _gpu_all(K, a_int8, a_scale, w_mx, w_sc, dump)
    o0 = orc.run_o0(a_int8, a_scale, w_mx, w_sc)["output"]
    o1 = orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"]
    o2 = orc.run_o2(a_int8, a_scale, w_mx, w_sc)["output"]
    if dump:
        np.testing.assert_array_equal(partials, orc.o1_partials(a_int8, orc.mxfp4_to_int8_base(w_mx)))
    np.testing.assert_allclose(y0, o0, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(y1, o1, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(y2, o2, rtol=RTOL, atol=ATOL)
    np.testing.assert_array_equal(y1, o1)
    for got, want in ((orc.mse_fp64(y1, y0), orc.mse_fp64(o1, o0)), (orc.mse_fp64(y2, y0), orc.mse_fp64(o2, o0))):
        assert got == pytest.approx(want, rel=0.02, abs=1e-12)
    return y0, y1, y2


def test_layout_probe():
    from adangel_oyzl_b200.ops import _sm100

    result = _sm100.verify_layout()
    assert result["passed"], result
    assert result["max_abs_error"] <= 1e-3


@pytest.mark.parametrize("name", GOLDEN)
def test_golden_files(K, golden_dir, name):
    ref, args = golden_inputs(golden_dir, name)
    y0, y1, y2 = _compare(K, *args)
    # and against the reference's own stored outputs
    np.testing.assert_allclose(y0, ref["o0_output"], rtol=RTOL, atol=ATOL)
    np.testing.assert_array_equal(y1, ref["o1_output"])
    np.testing.assert_allclose(y2, ref["o2_output"], rtol=RTOL, atol=ATOL)
    assert orc.mse_fp64(y1, y0) == pytest.approx(float(ref["mse_o1"]), rel=0.02, abs=1e-12)
    assert orc.mse_fp64(y2, y0) == pytest.approx(float(ref["mse_o2"]), rel=0.02, abs=1e-12)


@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 512, 1024), (1000, 768, 2048)])
def test_canonical_grid(K, shape):
    _compare(K, *orc.canonical_inputs(*shape), dump=shape[0] <= 256)


@pytest.mark.parametrize("shape", [(1, 128, 64), (16, 256, 192), (64, 384, 320), (129, 257 * 4, 448), (300, 40, 128),
                                   (5, 4096, 1024), (48, 136, 2048), (33, 128, 4096)])
def test_ragged_shapes(K, shape):
    # K not a multiple of the kernels' K slab, M/N not multiples of the tile, single-row A
    m, n, k = shape
    _compare(K, *orc.canonical_inputs(m, n, k, seed=11))


@pytest.mark.parametrize("shape", [(1, 128, 64), (16, 256, 192), (17, 200, 320), (64, 384, 320), (5, 4096, 1024),
                                   (48, 136, 2048), (33, 128, 4096), (64, 1024, 4096), (64, 4992, 256), (33, 9600, 128)])
def test_decode_shapes(K, shape):
    # M <= 64 without the partial dump: the operand-swapped O1 and O2 kernels (the last two shapes: more CTAs than SMs)
    m, n, k = shape
    _compare(K, *orc.canonical_inputs(m, n, k, seed=13), dump=False)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (2, 100, 192), (3, 9600, 256), (4, 352, 4160), (7, 4800, 640),
                                   (8, 64, 2048), (9, 4736, 192), (13, 31, 1088), (16, 4704, 4096)])
def test_o1_decode_ring_shapes(K, shape):
    # M <= 16: the dp4a kernel whose warps take the K slabs in turn -- every rows-per-thread variant, both
    # ring sizes (N / 32 above and below what is resident at once), one, few and many turns, ragged K and N
    import torch

    m, n, k = shape
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(m, n, k, seed=29)
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    y = torch.full((m, n), float("nan"), device="cuda")
    K.gemm_o1(da, ds, K.mxfp4_to_int8(dw), dws, out=y)
    K.check_status()
    want = orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"]
    np.testing.assert_array_equal(y.cpu().numpy(), want)
    # the same kernel reading the packed MXFP4 weights themselves
    y.fill_(float("nan"))
    K.gemm_o1_packed(da, ds, dw, dws, out=y)
    K.check_status()
    np.testing.assert_array_equal(y.cpu().numpy(), want)


def test_o1_packed_refuses_shapes_of_the_tile_kernels(K):
    import torch

    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(40, 128, 128, seed=2)
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    with pytest.raises(RuntimeError, match="decode kernel"):
        K.gemm_o1_packed(da, ds, dw, dws)


def test_decode_matches_prefill_rows(K):
    # the decode kernels and the 128-row-tile kernels give the same bits for the same activation rows
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(160, 512, 1024, seed=17)
    full = _gpu_all(K, a_int8, a_scale, w_mx, w_sc)
    part = _gpu_all(K, a_int8[:40], a_scale[:40], w_mx, w_sc)
    np.testing.assert_array_equal(part[1], full[1][:40])
    np.testing.assert_allclose(part[2], full[2][:40], rtol=RTOL, atol=ATOL)


def test_output_column_block(K):
    # Y written as a column block of a wider matrix (the N-sharded layout): ldy > N
    import torch

    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(200, 384, 256, seed=5)
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    wide = torch.full((200, 1024), -7.0, device="cuda")
    K.gemm_o0(K.int8_to_fp16(da, ds), K.mxfp4_to_fp16(dw, dws), out=wide[:, 128:512])
    K.gemm_o1(da, ds, K.mxfp4_to_int8(dw), dws, out=wide[:, 512:896])
    K.check_status()
    got = wide.cpu().numpy()
    np.testing.assert_allclose(got[:, 128:512], orc.run_o0(a_int8, a_scale, w_mx, w_sc)["output"], rtol=RTOL, atol=ATOL)
    np.testing.assert_array_equal(got[:, 512:896], orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"])
    assert (got[:, :128] == -7.0).all() and (got[:, 896:] == -7.0).all()


def test_deterministic_rerun(K):
    # the same launch twice must give the same bits (a difference would indicate a race)
    args = orc.canonical_inputs(384, 512, 512, seed=3)
    first = _gpu_all(K, *args)
    second = _gpu_all(K, *args)
    for a, b in zip(first[:3], second[:3]):
        np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 320), (1000, 777, 128), (4224, 512, 256)])
def test_cta_pair_kernels_match_single_cta(K, shape, monkeypatch):
    # O0/O2 on CTA pairs (cta_group::2, the default for large shapes) give the
    # same bits as the single-CTA kernels; (1000, 777, .) has ragged edges and an unaligned Y pitch,
    # (4224, ...) an odd number of row blocks
    m, n, k = shape
    args = orc.canonical_inputs(m, n, k, seed=23)
    monkeypatch.setenv("ADG_TWO_CTA", "0")
    single = _gpu_all(K, *args)
    monkeypatch.setenv("ADG_TWO_CTA", "1")  # pairs wherever a full pair tile exists, not only where they pay
    paired = _gpu_all(K, *args)
    np.testing.assert_array_equal(paired[0], single[0])
    np.testing.assert_array_equal(paired[2], single[2])
    np.testing.assert_allclose(paired[0], orc.run_o0(*args)["output"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("shape", [(128, 128, 64), (200, 384, 256), (1000, 777, 128), (512, 1024, 2048)])
def test_o1_bf16_operands_bit_identical(K, shape):
    # the O1 kernel that takes the weight scale through the tensor core (BF16 operands) gives the
    # oracle's bits, like the INT8-operand kernel
    m, n, k = shape
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(m, n, k, seed=29)
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    flag = K.new_range_flag("cuda")
    y = K.gemm_o1_bf16(K.int8_to_bf16(da, ds, flag), ds, K.mxfp4_to_bf16_scaled(dw, dws, flag), flag)
    K.check_status()
    assert int(flag.item()) == 0
    np.testing.assert_array_equal(y.cpu().numpy(), orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"])


def test_o1_bf16_operands_refuse_out_of_range(K):
    # scale codes / activation scales outside the exact range set the flag; the GEMM then refuses
    # loudly instead of returning different bits, and the INT8-operand kernel still serves the input
    import torch

    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(128, 128, 128, seed=31)
    w_sc = w_sc.copy()
    w_sc[5, 1] = 250
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    flag = K.new_range_flag("cuda")
    wb = K.mxfp4_to_bf16_scaled(dw, dws, flag)
    ab = K.int8_to_bf16(da, ds, flag)
    assert int(flag.item()) == 1
    y = torch.full((128, 128), -3.0, device="cuda")
    K.gemm_o1_bf16(ab, ds, wb, flag, out=y)
    with pytest.raises(RuntimeError, match="outside its exact range"):
        K.check_status()
    assert bool((y == -3.0).all())
    K.check_status()  # the error is reported once
    flag2 = K.new_range_flag("cuda")
    tiny = ds.clone()
    tiny[7] = 1e-30
    K.int8_to_bf16(da, tiny, flag2)
    assert int(flag2.item()) == 2
    y1 = K.gemm_o1(da, ds, K.mxfp4_to_int8(dw), dws)
    K.check_status()
    np.testing.assert_array_equal(y1.cpu().numpy(), orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"])


def test_cta_pair_output_column_block(K, monkeypatch):
    # pair-tile shapes writing Y as a column block of a wider matrix (ldy > N), O0 and O2
    import torch

    monkeypatch.setenv("ADG_TWO_CTA", "1")

    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(512, 256, 256, seed=37)
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    wide = torch.full((512, 1024), -7.0, device="cuda")
    K.gemm_o0(K.int8_to_fp16(da, ds), K.mxfp4_to_fp16(dw, dws), out=wide[:, 128:384])
    codes, _, sfa = K.o2_quantize_activation(da, ds)
    K.gemm_o2(codes, sfa, dw, K.o2_tile_scales(dws), out=wide[:, 640:896])
    K.check_status()
    got = wide.cpu().numpy()
    np.testing.assert_allclose(got[:, 128:384], orc.run_o0(a_int8, a_scale, w_mx, w_sc)["output"], rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(got[:, 640:896], orc.run_o2(a_int8, a_scale, w_mx, w_sc)["output"], rtol=RTOL, atol=ATOL)
    untouched = np.ones(1024, dtype=bool)
    untouched[128:384] = untouched[640:896] = False
    assert (got[:, untouched] == -7.0).all()


def test_o1_linear_every_input_without_sync(K):
    # adg_o1_linear: the BF16-operand kernel, and behind it the INT8-operand kernel that runs only if the first
    # refused; oracle bits for in-range operands, for an out-of-range activation scale, for an out-of-range
    # weight scale code and for decode-sized M, and never an error status
    import torch

    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(320, 384, 512, seed=47)
    odd_a = a_scale.copy()
    odd_a[11] = np.float32(2.0 ** -50)
    odd_w = w_sc.copy()
    odd_w[17, 3] = 240
    for scale_a, scale_w, rows in ((a_scale, w_sc, 320), (odd_a, w_sc, 320), (a_scale, odd_w, 320), (a_scale, w_sc, 48)):
        da, ds, dw, dws = to_cuda(a_int8[:rows], scale_a[:rows], w_mx, scale_w)
        weights = K.O1Weights(dw, dws)
        y = torch.full((rows, 384), float("nan"), device="cuda")
        for _ in range(2):  # the per-call flag word is rebuilt on every call
            K.o1_linear(da, ds, weights, out=y)
        K.check_status()
        np.testing.assert_array_equal(y.cpu().numpy(), orc.run_o1(a_int8[:rows], scale_a[:rows], w_mx, scale_w)["output"])
