"""Parity of the conversion kernels with the CPU oracle, through the C ABI.  Bit-exact."""

import numpy as np
import pytest

from oracle import adangel_oracle as orc
from tests.gpu_util import assert_requant_matches, golden_inputs, to_cuda

pytestmark = pytest.mark.gpu

GRID = [(128, 128, 128), (256, 512, 1024), (1000, 768, 2048)]
GOLDEN = ["canonical_128x128x128", "canonical_68x36x64", "fp16_seed2026_132x132x256",
          "edge_zero_128x128x256", "edge_alternating_128x128x256", "edge_saturated_128x128x256", "seed7_16x8x64"]


@pytest.fixture(scope="module")
def K():
    from adangel_oyzl_b200 import kernels

    return kernels


def _check_all(K, a_int8, a_scale, w_mx, w_sc):
    da, ds, dw, dws = to_cuda(a_int8, a_scale, w_mx, w_sc)
    w16 = K.mxfp4_to_fp16(dw, dws).cpu().numpy()
    a16 = K.int8_to_fp16(da, ds).cpu().numpy()
    w8 = K.mxfp4_to_int8(dw).cpu().numpy()
    codes, nat, tiled = K.o2_quantize_activation(da, ds)
    wtiled = K.o2_tile_scales(dws).cpu().numpy()
    K.check_status()
    np.testing.assert_array_equal(w16.view(np.uint16), orc.dequantize_mxfp4(w_mx, w_sc, np.float16).view(np.uint16))
    np.testing.assert_array_equal(a16.view(np.uint16), orc.dequantize_int8_per_row(a_int8, a_scale, np.float16).view(np.uint16))
    np.testing.assert_array_equal(w8, orc.mxfp4_to_int8_base(w_mx))
    assert_requant_matches(codes.cpu().numpy(), nat.cpu().numpy(), a_int8, a_scale, orc)
    np.testing.assert_array_equal(tiled.cpu().numpy(), orc.tile_scale_factors(nat.cpu().numpy()))
    np.testing.assert_array_equal(wtiled, orc.tile_scale_factors(w_sc))


@pytest.mark.parametrize("shape", GRID)
def test_canonical_grid(K, shape):
    _check_all(K, *orc.canonical_inputs(*shape))


@pytest.mark.parametrize("name", GOLDEN)
def test_golden_files(K, golden_dir, name):
    ref, args = golden_inputs(golden_dir, name)
    _check_all(K, *args)
    # and against the stored outputs of the reference itself
    da, ds, dw, dws = to_cuda(*args)
    np.testing.assert_array_equal(K.mxfp4_to_fp16(dw, dws).cpu().numpy().view(np.uint16), ref["o0_weight"].view(np.uint16))
    np.testing.assert_array_equal(K.int8_to_fp16(da, ds).cpu().numpy().view(np.uint16), ref["o0_activation"].view(np.uint16))
    np.testing.assert_array_equal(K.mxfp4_to_int8(dw).cpu().numpy(), ref["o1_weight"])
    codes, nat, _ = K.o2_quantize_activation(da, ds)
    np.testing.assert_array_equal(codes.cpu().numpy(), ref["o2_codes"])
    np.testing.assert_array_equal(nat.cpu().numpy(), ref["o2_scales"])


def test_weight_dequant_all_scale_codes(K):
    # every nibble value under every finite UE8M0 code: overflow to inf, FP16 subnormals, underflow
    codes = np.arange(255, dtype=np.uint8)
    w_sc = np.repeat(codes[:, None], 2, axis=1)  # [255, 2] -> K = 64
    nibbles = np.arange(16, dtype=np.uint8)
    row = np.tile(nibbles | (nibbles[::-1] << 4), 2)  # 32 bytes = 64 elements
    w_mx = np.tile(row, (255, 1))
    dw, dws = to_cuda(w_mx, w_sc)
    got = K.mxfp4_to_fp16(dw, dws).cpu().numpy()
    want = orc.dequantize_mxfp4(w_mx, w_sc, np.float16)
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))


def test_activation_edge_scales(K):
    rng = np.random.default_rng(3)
    m, k = 96, 256
    a_int8 = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    a_int8[0] = 0
    a_int8[1, ::2] = 0
    a_scale = np.concatenate([
        np.float32(2.0) ** np.arange(-40, 40, dtype=np.float32)[:80],
        np.array([-1.0, -0.0, 0.0, 1e-38, 3e38 / 127, 1.0, 0.1, 7.3, 1e-30, 1e30, 2.5e-39, 1.0, 1.0, 1.0, 1.0, 1.0], dtype=np.float32),
    ]).astype(np.float32)
    assert a_scale.shape == (m,)
    da, ds = to_cuda(a_int8, a_scale)
    a16 = K.int8_to_fp16(da, ds).cpu().numpy()
    np.testing.assert_array_equal(a16.view(np.uint16), orc.dequantize_int8_per_row(a_int8, a_scale, np.float16).view(np.uint16))
    codes, nat, _ = K.o2_quantize_activation(da, ds)
    assert_requant_matches(codes.cpu().numpy(), nat.cpu().numpy(), a_int8, a_scale, orc)


def test_requant_near_power_of_two(K):
    # block maxima a few ulps around powers of two: the exponent must be the exact floor(log2)
    m, k = 64, 64
    a_int8 = np.zeros((m, k), dtype=np.int8)
    a_int8[:, 0] = 127
    a_int8[:, 40] = 64
    base = np.float32(2.0) ** np.arange(-16, 16, dtype=np.float32)
    scales = []
    for b in base:
        s = np.float32(b / np.float32(127.0))
        scales += [np.nextafter(s, np.float32(0)), np.nextafter(s, np.float32(np.inf))]
    a_scale = np.array(scales, dtype=np.float32)
    da, ds = to_cuda(a_int8, a_scale)
    codes, nat, _ = K.o2_quantize_activation(da, ds)
    assert_requant_matches(codes.cpu().numpy(), nat.cpu().numpy(), a_int8, a_scale, orc)


def test_full_size_conversion_properties(K):
    """4096x4096 operands: checked through size-independent properties and sampled rows."""
    import torch

    from adangel_oyzl_b200 import synthetic

    p = synthetic.canonical_inputs(4096, 4096, 4096, device="cuda")
    w8 = K.mxfp4_to_int8(p.W_mxfp4)
    w16 = K.mxfp4_to_fp16(p.W_mxfp4, p.W_scale)
    a16 = K.int8_to_fp16(p.A_int8, p.A_scale)
    codes, nat, tiled = K.o2_quantize_activation(p.A_int8, p.A_scale)
    K.check_status()
    # 2*E2M1 image: w16 == w8 * 2^(s-128) exactly wherever that product is a normal half
    exps = p.W_scale.to(torch.int32) - 128
    scale = torch.ldexp(torch.ones_like(exps, dtype=torch.float32), exps)
    recon = (w8.float().reshape(4096, 128, 32) * scale[:, :, None]).reshape(4096, 4096)
    assert torch.equal(recon.half(), w16)
    # dequantize(requantize(A)) stays within half an E2M1 step of A in every block
    rows = torch.arange(0, 4096, 61, device="cuda")
    a_np, s_np = p.A_int8[rows].cpu().numpy(), p.A_scale[rows].cpu().numpy()
    assert_requant_matches(codes[rows].cpu().numpy(), nat[rows].cpu().numpy(), a_np, s_np, orc)
    np.testing.assert_array_equal(a16[rows].cpu().numpy().view(np.uint16),
                                  orc.dequantize_int8_per_row(a_np, s_np, np.float16).view(np.uint16))
    w_np, ws_np = p.W_mxfp4[rows].cpu().numpy(), p.W_scale[rows].cpu().numpy()
    np.testing.assert_array_equal(w16[rows].cpu().numpy().view(np.uint16), orc.dequantize_mxfp4(w_np, ws_np, np.float16).view(np.uint16))
    np.testing.assert_array_equal(w8[rows].cpu().numpy(), orc.mxfp4_to_int8_base(w_np))
    np.testing.assert_array_equal(tiled.cpu().numpy(), orc.tile_scale_factors(nat.cpu().numpy()))
