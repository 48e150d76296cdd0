"""The numpy oracle must reproduce every golden vector produced by the reference's own code."""

import hashlib
import json

import numpy as np
import pytest

from oracle import adangel_oracle as orc

FULL_CASES = [
    "canonical_128x128x128",
    "canonical_68x36x64",
    "fp16_seed2026_128x128x256",
    "fp16_seed2026_132x132x256",
    "edge_zero_128x128x256",
    "edge_alternating_128x128x256",
    "edge_saturated_128x128x256",
    "seed7_16x8x64",
]


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_scalar_known_answers(golden_dir):
    ref = json.loads((golden_dir / "scalar_codec.json").read_text())
    values = np.array(ref["encode_values"], dtype=np.float64).astype(np.float32)
    assert orc.encode_e2m1(values).tolist() == ref["encode_codes"]
    assert orc.decode_e2m1(np.arange(16)).tolist() == ref["decode"]
    assert orc.E2M1_TO_INT8_BASE.tolist() == ref["int8_base"]
    assert orc.pack_e2m1(np.array([1, 2], dtype=np.uint8)).tolist() == ref["pack_1_2"] == [0x21]
    amax = np.array([float.fromhex(h) for h in ref["scale_inputs"]], dtype=np.float32)
    assert (orc.block_exponent(amax) + 127).tolist() == ref["scale_codes"]


def test_reference_unit_table():
    # reference tests/unit/test_mxfp4_codec.py:26-52
    ties = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6}
    for value, code in ties.items():
        assert int(orc.encode_e2m1(np.float32(value))) == code
        assert int(orc.encode_e2m1(np.float32(-value))) == code | 8
    assert int(orc.encode_e2m1(np.float32(100.0))) == 7
    assert int(orc.encode_e2m1(np.float32(-100.0))) == 15
    assert int(orc.encode_e2m1(np.float32(-0.0))) == 0
    assert float(orc.decode_ue8m0(np.array([127], dtype=np.uint8))[0]) == 1.0
    for amax, code in ((0.0, 127), (4.0, 127), (8.0, 128)):
        assert int(orc.block_exponent(np.float32(amax))) + 127 == code
    with pytest.raises(ValueError):
        orc.decode_ue8m0(np.array([255], dtype=np.uint8))
    with pytest.raises(ValueError):
        orc.quantize_mxfp4(np.full((1, 32), np.nan, dtype=np.float32))


def test_seed7_quantizers(golden_dir):
    floats = np.load(golden_dir / "seed7_floats.npz")
    ref = np.load(golden_dir / "seed7_16x8x64.npz")
    a_int8, a_scale = orc.quantize_int8_per_row(floats["a"])
    w_mx, w_sc = orc.quantize_mxfp4(floats["w"])
    np.testing.assert_array_equal(a_int8, ref["A_int8"])
    np.testing.assert_array_equal(a_scale, ref["A_scale"])
    np.testing.assert_array_equal(w_mx, ref["W_mxfp4"])
    np.testing.assert_array_equal(w_sc, ref["W_scale"])


@pytest.mark.parametrize("name", FULL_CASES)
def test_full_cases(golden_dir, name):
    ref = np.load(golden_dir / f"{name}.npz")
    args = (ref["A_int8"], ref["A_scale"], ref["W_mxfp4"], ref["W_scale"])
    o0 = orc.run_o0(*args)
    o1 = orc.run_o1(*args)
    o2 = orc.run_o2(*args)
    # conversions, codes, scales: bit-exact
    np.testing.assert_array_equal(o0["converted_weight"].view(np.uint16), ref["o0_weight"].view(np.uint16))
    np.testing.assert_array_equal(o0["converted_activation"].view(np.uint16), ref["o0_activation"].view(np.uint16))
    np.testing.assert_array_equal(o1["converted_weight"], ref["o1_weight"])
    np.testing.assert_array_equal(o2["converted_activation"][0], ref["o2_codes"])
    np.testing.assert_array_equal(o2["converted_activation"][1], ref["o2_scales"])
    # FP32 outputs: same tolerance the reference's tests use (rtol = atol = 1e-3)
    np.testing.assert_allclose(o0["output"], ref["o0_output"], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(o1["output"], ref["o1_output"], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(o2["output"], ref["o2_output"], rtol=1e-3, atol=1e-3)
    # O1 follows the same operation order as the reference, so it is bit-identical
    np.testing.assert_array_equal(o1["output"], ref["o1_output"])
    # INT32 partials agree between the einsum form and the per-group FP32 form used by run_o1
    w_int8 = o1["converted_weight"]
    p = orc.o1_partials(args[0], w_int8)
    g0 = args[0][:, :32].astype(np.float32) @ w_int8[:, :32].astype(np.float32).T
    np.testing.assert_array_equal(p[:, :, 0], g0.astype(np.int32))
    for key, mine in (("mse_o1", orc.mse_fp64(o1["output"], o0["output"])),
                      ("mse_o2", orc.mse_fp64(o2["output"], o0["output"]))):
        want = float(ref[key])
        assert mine == pytest.approx(want, rel=0.02, abs=1e-12)


@pytest.mark.parametrize("shape", [(256, 512, 1024), (1000, 768, 2048)])
def test_canonical_generator_digests(golden_dir, shape):
    m, n, k = shape
    key = f"{m}x{n}x{k}"
    want = json.loads((golden_dir / "canonical_digests.json").read_text())[key]
    sample = np.load(golden_dir / f"canonical_{key}_sample.npz")
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(m, n, k)
    assert _sha(a_int8) == want["A_int8"]
    assert _sha(a_scale) == want["A_scale"]
    assert _sha(w_mx) == want["W_mxfp4"]
    assert _sha(w_sc) == want["W_scale"]
    o0 = orc.run_o0(a_int8, a_scale, w_mx, w_sc)
    o1 = orc.run_o1(a_int8, a_scale, w_mx, w_sc)
    o2 = orc.run_o2(a_int8, a_scale, w_mx, w_sc)
    assert _sha(o0["converted_weight"]) == want["o0_weight"]
    assert _sha(o0["converted_activation"]) == want["o0_activation"]
    assert _sha(o1["converted_weight"]) == want["o1_weight"]
    assert _sha(o2["converted_activation"][0]) == want["o2_codes"]
    assert _sha(o2["converted_activation"][1]) == want["o2_scales"]
    np.testing.assert_allclose(o0["output"][::8, ::8], sample["o0"], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(o1["output"][::8, ::8], sample["o1"], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(o2["output"][::8, ::8], sample["o2"], rtol=1e-3, atol=1e-3)
    assert orc.mse_fp64(o1["output"], o0["output"]) == pytest.approx(want["mse_o1"], rel=0.02)
    assert orc.mse_fp64(o2["output"], o0["output"]) == pytest.approx(want["mse_o2"], rel=0.02)


def test_exponent_hazard_is_classified():
    # just below a power of two the FP32-log2 exponent may exceed the exact one by exactly one
    amax = np.nextafter(np.float32(2.0) ** np.arange(-20, 21, dtype=np.float32), np.float32(0))
    exact = orc.block_exponent(amax)
    loose = orc.block_exponent_log2_fp32(amax)
    assert ((loose == exact) | (loose == exact + 1)).all()
    rnd = np.random.default_rng(0).standard_normal(200000).astype(np.float32)
    np.testing.assert_array_equal(orc.block_exponent(np.abs(rnd)), orc.block_exponent_log2_fp32(np.abs(rnd)))


def test_tiled_scale_layout_roundtrip():
    rng = np.random.default_rng(1)
    nat = rng.integers(0, 255, size=(132, 10), dtype=np.uint8)
    tiled = orc.tile_scale_factors(nat)
    prow, pgroups = orc.tiled_scale_shape(132, 320)
    assert tiled.size == prow * pgroups
    for r, g in ((0, 0), (31, 3), (32, 0), (127, 9), (128, 4), (131, 7)):
        off = ((r // 128) * (pgroups // 4) + g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + g % 4
        assert tiled[off] == nat[r, g]
    assert int(tiled.astype(np.int64).sum()) == int(nat.astype(np.int64).sum())
