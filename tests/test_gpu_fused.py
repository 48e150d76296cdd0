"""The one-kernel steady-state passes of O0 and O2 (activation conversion done by converter warps inside
the GEMM kernel, ``adg_o0_linear`` / ``adg_o2_linear``) against the two-kernel sequence they replace:
the converted operand left in the workspace and the output must be bit-identical, on single-CTA and
CTA-pair kernels, ragged shapes, repeated calls on the same counters and the decode-size fallback.
The two-kernel sequence itself is compared with the oracle in test_gpu_gemm.py.
"""

import numpy as np
import pytest

from oracle import adangel_oracle as orc
from tests.gpu_util import to_cuda

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-3


@pytest.fixture(scope="module")
def K():
    from adangel_oyzl_b200 import kernels

    return kernels


def _both(K, a_int8, a_scale, w_mx, w_sc, calls=2):
    import torch

    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    m, k = a_int8.shape
    w16 = K.mxfp4_to_fp16(dw, dws)
    wsf = K.o2_tile_scales(dws)
    a16 = K.int8_to_fp16(da, ds)
    y0 = K.gemm_o0(a16, w16)
    codes, nat, sfa = K.o2_quantize_activation(da, ds)
    y2 = K.gemm_o2(codes, sfa, dw, wsf)
    ws0 = K.FusedWorkspace("o0", m, k, da.device, fuse=True)
    ws2 = K.FusedWorkspace("o2", m, k, da.device, want_natural_scales=True, fuse=True)
    for _ in range(calls):  # the kernels must leave their row counters zero for the next call
        f0 = K.o0_linear(da, ds, w16, ws0)
        f2 = K.o2_linear(da, ds, dw, wsf, ws2)
    K.check_status()
    assert int(ws0.counters.abs().sum().item()) == 0 and int(ws2.counters.abs().sum().item()) == 0
    assert torch.equal(ws0.operand[:m].view(torch.int16), a16.view(torch.int16))
    assert torch.equal(ws2.operand[:m], codes)
    assert torch.equal(ws2.sf_natural[:m], nat)
    assert torch.equal(ws2.sf_tiled, sfa)
    assert torch.equal(f0, y0)
    assert torch.equal(f2, y2)
    return f0.cpu().numpy(), f2.cpu().numpy()


@pytest.mark.parametrize("shape", [(200, 384, 512), (1000, 777, 128), (300, 256, 192), (512, 1024, 2048), (129, 1028, 448),
                                   (2048, 512, 11008)])
def test_fused_matches_two_kernel_sequence(K, shape, monkeypatch):
    m, n, k = shape
    args = orc.canonical_inputs(m, n, k, seed=41)
    f0, f2 = _both(K, *args)
    if m * n * k <= 512 * 1024 * 2048:
        np.testing.assert_allclose(f0, orc.run_o0(*args)["output"], rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(f2, orc.run_o2(*args)["output"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("shape", [(512, 768, 320), (1000, 777, 128), (4224, 512, 256)])
def test_fused_on_cta_pairs(K, shape, monkeypatch):
    # pairs wherever a full pair tile exists; (4224, ...) has an odd number of row blocks, so the last
    # pair's second CTA has no rows to wait for
    from adangel_oyzl_b200.ops import _sm100

    monkeypatch.setenv("ADG_TWO_CTA", "1")
    m, n, k = shape
    assert _sm100.plan_info("o2", m, n, k, fused=True)["kernel_symbol"] == "gemm_pair_kernel<2,fused>"
    _both(K, *orc.canonical_inputs(m, n, k, seed=43))


def test_fused_canonical_4096(K, monkeypatch):
    # the benchmarked shape: O0 on CTA pairs, O2 on single CTAs (the planner's own choice)
    import torch

    from adangel_oyzl_b200 import synthetic

    monkeypatch.delenv("ADG_TWO_CTA", raising=False)
    p = synthetic.canonical_inputs(4096, 4096, 4096, device="cuda")
    w16, wsf = K.mxfp4_to_fp16(p.W_mxfp4, p.W_scale), K.o2_tile_scales(p.W_scale)
    y0 = K.gemm_o0(K.int8_to_fp16(p.A_int8, p.A_scale), w16)
    codes, _, sfa = K.o2_quantize_activation(p.A_int8, p.A_scale)
    y2 = K.gemm_o2(codes, sfa, p.W_mxfp4, wsf)
    ws0, ws2 = K.FusedWorkspace("o0", 4096, 4096, "cuda", fuse=True), K.FusedWorkspace("o2", 4096, 4096, "cuda", fuse=True)
    for _ in range(3):
        f0 = K.o0_linear(p.A_int8, p.A_scale, w16, ws0)
        f2 = K.o2_linear(p.A_int8, p.A_scale, p.W_mxfp4, wsf, ws2)
    K.check_status()
    assert torch.equal(f0, y0) and torch.equal(f2, y2)
    assert torch.equal(ws2.operand, codes) and torch.equal(ws2.sf_tiled, sfa)


def test_decode_sizes_and_default_take_two_kernels(K):
    # M <= 64 (the decode kernels convert nothing themselves) with counters given, and the default workspace
    # without counters at a larger M: the two-kernel sequence behind the same entry points, same results
    import torch

    args = orc.canonical_inputs(48, 256, 512, seed=47)
    _both(K, *args, calls=1)
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(320, 256, 512, seed=47)
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    ws0, ws2 = K.FusedWorkspace("o0", 320, 512, "cuda"), K.FusedWorkspace("o2", 320, 512, "cuda")
    assert ws0.counters is None and ws2.counters is None
    w16, wsf = K.mxfp4_to_fp16(dw, dws), K.o2_tile_scales(dws)
    y0, y2 = K.o0_linear(da, ds, w16, ws0), K.o2_linear(da, ds, dw, wsf, ws2)
    K.check_status()
    codes, _, sfa = K.o2_quantize_activation(da, ds)
    assert torch.equal(y0, K.gemm_o0(K.int8_to_fp16(da, ds), w16)) and torch.equal(y2, K.gemm_o2(codes, sfa, dw, wsf))


def test_fused_output_column_block(K):
    # Y as a column block of a wider matrix (the N-sharded layout)
    import torch

    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(384, 256, 512, seed=53)
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    wide = torch.full((384, 1024), -7.0, device="cuda")
    K.o0_linear(da, ds, K.mxfp4_to_fp16(dw, dws), K.FusedWorkspace("o0", 384, 512, "cuda", fuse=True), out=wide[:, 128:384])
    K.o2_linear(da, ds, dw, K.o2_tile_scales(dws), K.FusedWorkspace("o2", 384, 512, "cuda", fuse=True), out=wide[:, 640:896])
    K.check_status()
    got = wide.cpu().numpy()
    np.testing.assert_allclose(got[:, 128:384], orc.run_o0(a_int8, a_scale, w_mx, w_sc)["output"], rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(got[:, 640:896], orc.run_o2(a_int8, a_scale, w_mx, w_sc)["output"], rtol=RTOL, atol=ATOL)
    untouched = np.ones(1024, dtype=bool)
    untouched[128:384] = untouched[640:896] = False
    assert (got[:, untouched] == -7.0).all()
