"""The reference-facing ops surface on a GPU: dispatch, timing-mode contract, error behaviour.

Follows the reference's integration tests (tests/integration/test_sm120_o0.py:25-85,
test_sm120_o1.py:25-128, test_sm120_o2.py:31-185) with the metadata asserts re-targeted to sm_100a.
"""

import subprocess
import sys

import numpy as np
import pytest

from oracle import adangel_oracle as orc
from tests.gpu_util import golden_inputs

pytestmark = pytest.mark.gpu


def _prepared(golden_dir, name="fp16_seed2026_128x128x256"):
    import torch

    from adangel_oyzl_b200.schema import PreparedInputs

    ref, args = golden_inputs(golden_dir, name)
    cuda = PreparedInputs("golden", *(torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in args))
    return ref, args, cuda


def test_doctor_require_native():
    out = subprocess.run([sys.executable, "-m", "adangel_oyzl_b200", "doctor", "--require-native"],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert '"available": true' in out.stdout


def test_run_variants_match_oracle(golden_dir):
    import torch

    from adangel_oyzl_b200.ops import run_o0, run_o1, run_o2

    ref, args, cuda = _prepared(golden_dir)
    r0 = run_o0(cuda, mode="compute_only")
    r1 = run_o1(cuda, mode="compute_only")
    r2 = run_o2(cuda, mode="compute_only")
    torch.cuda.synchronize()
    # O0: converted operands bit-exact, output within tolerance
    np.testing.assert_array_equal(r0["converted_activation"].cpu().numpy().view(np.uint16), ref["o0_activation"].view(np.uint16))
    np.testing.assert_array_equal(r0["converted_weight"].cpu().numpy().view(np.uint16), ref["o0_weight"].view(np.uint16))
    np.testing.assert_allclose(r0["output"].cpu().numpy(), ref["o0_output"], rtol=1e-3, atol=1e-3)
    # O1
    np.testing.assert_array_equal(r1["converted_weight"].cpu().numpy(), ref["o1_weight"])
    assert r1["converted_activation"] is None
    np.testing.assert_allclose(r1["output"].cpu().numpy(), ref["o1_output"], rtol=1e-3, atol=1e-3)
    # O2
    values, scales = r2["converted_activation"]
    np.testing.assert_array_equal(values.cpu().numpy(), ref["o2_codes"])
    np.testing.assert_array_equal(scales.cpu().numpy(), ref["o2_scales"])
    assert r2["converted_weight"] is None
    np.testing.assert_allclose(r2["output"].cpu().numpy(), ref["o2_output"], rtol=1e-3, atol=1e-3)
    for r in (r0, r1, r2):
        assert r["output"].dtype == torch.float32 and torch.isfinite(r["output"]).all()
        kernel = dict(r["kernel"])
        assert kernel["tensor_core"] is True
        assert kernel["data_movement"] == "TMA"
        assert kernel["global_partial_buffer"] is False
        assert kernel["output_stores_per_element"] == 1
        assert kernel["group_size"] == 32
        assert kernel["mma_family"].startswith("tcgen05.mma")
        for key in ("weight_conversion_ms", "activation_conversion_ms", "gemm_ms", "total_ms"):
            assert key in r


@pytest.mark.parametrize("variant", ["o0", "o1", "o2"])
@pytest.mark.parametrize("mode", ["conversion_only", "compute_only", "cold", "steady_state"])
def test_timing_mode_contract(golden_dir, variant, mode):
    from adangel_oyzl_b200.ops.extension import require_variant

    _, _, cuda = _prepared(golden_dir)
    native = require_variant(variant)
    result = native.benchmark(variant, mode, cuda.A_int8, cuda.A_scale, cuda.W_mxfp4, cuda.W_scale, 2, 3)
    # the reference's stage sets (tests/integration/test_sm120_o{0,1,2}.py): O1 never has an activation stage --
    # on BF16 operands its INT8 -> BF16 conversion is part of this build's gemm stage unless asked otherwise
    has_act = variant != "o1"
    expected = {
        "conversion_only": {"weight_conversion", "total"} | ({"activation_conversion"} if has_act else set()),
        "compute_only": {"gemm", "total"},
        "cold": {"weight_conversion", "gemm", "total"} | ({"activation_conversion"} if has_act else set()),
        "steady_state": {"gemm", "total"} | ({"activation_conversion"} if has_act else set()),
    }[mode]
    assert set(result["timings_ms"]) == expected
    for values in result["timings_ms"].values():
        assert len(values) == 3 and all(v > 0 for v in values)
    method = result["timing_method"]
    assert method["strategy"] == "conversion_amortized_end_to_end_direct"
    assert method["conversion_inner_repeats"] == 100
    assert method["mode_total_timing"] == ("batched_cuda_event_average" if mode == "conversion_only" else "direct_single_path")
    want = {"o0": orc.run_o0, "o1": orc.run_o1, "o2": orc.run_o2}[variant]
    args = tuple(t.cpu().numpy() for t in (cuda.A_int8, cuda.A_scale, cuda.W_mxfp4, cuda.W_scale))
    np.testing.assert_allclose(result["output"].cpu().numpy(), want(*args)["output"], rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("variant", ["o0", "o2"])
@pytest.mark.parametrize("mode", ["cold", "steady_state"])
def test_harness_fused_and_separate_activation_paths_agree(variant, mode):
    # cold / steady_state of O0 and O2 run the reference's sequence of conversion kernel and GEMM (the default)
    # or, with fuse_activation=True, the GEMM kernel that converts A itself: same stages, same bits
    import torch

    from adangel_oyzl_b200.ops import _sm100

    args = orc.canonical_inputs(320, 384, 512, seed=71)
    dev = [torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in args]
    fused = _sm100.benchmark(variant, mode, *dev, 1, 2, 2, fuse_activation=True)
    plain = _sm100.benchmark(variant, mode, *dev, 1, 2, 2)
    assert fused["kernel"]["fused_activation_conversion"] and not plain["kernel"]["fused_activation_conversion"]
    assert set(fused["timings_ms"]) == set(plain["timings_ms"])
    assert torch.equal(fused["output"], plain["output"])
    if variant == "o2":
        for got, want in zip(fused["converted_activation"], plain["converted_activation"]):
            assert torch.equal(got, want)
    else:
        assert torch.equal(fused["converted_activation"].view(torch.int16), plain["converted_activation"].view(torch.int16))


def test_rejections(golden_dir):
    import torch

    from adangel_oyzl_b200.ops import _sm100
    from adangel_oyzl_b200.ops.dispatch import run_o2
    from adangel_oyzl_b200.schema import PreparedInputs

    _, _, cuda = _prepared(golden_dir)
    bad_scale = cuda.W_scale.clone()
    bad_scale[0, 0] = 255
    with pytest.raises(RuntimeError, match="UE8M0 NaN"):
        _sm100.run_o2(cuda.A_int8, cuda.A_scale, cuda.W_mxfp4, bad_scale, "cold")
    with pytest.raises(ValueError, match="UE8M0 NaN"):
        run_o2(PreparedInputs("bad", cuda.A_int8, cuda.A_scale, cuda.W_mxfp4, bad_scale))
    nan_scale = cuda.A_scale.clone()
    nan_scale[3] = float("nan")
    with pytest.raises(RuntimeError, match="A_scale contains NaN/Inf"):
        _sm100.run_o2(cuda.A_int8, nan_scale, cuda.W_mxfp4, cuda.W_scale, "cold")
    with pytest.raises(RuntimeError, match="unknown timing mode"):
        _sm100.benchmark("o0", "warm", cuda.A_int8, cuda.A_scale, cuda.W_mxfp4, cuda.W_scale, 0, 1)
    with pytest.raises(RuntimeError, match="not implemented"):
        _sm100.benchmark("o3", "cold", cuda.A_int8, cuda.A_scale, cuda.W_mxfp4, cuda.W_scale, 0, 1)
    with pytest.raises(RuntimeError, match="conversion_inner_repeats"):
        _sm100.benchmark("o0", "cold", cuda.A_int8, cuda.A_scale, cuda.W_mxfp4, cuda.W_scale, 0, 1, 1)
    with pytest.raises(RuntimeError, match="contiguous"):
        wide = torch.zeros((cuda.A_int8.shape[0], 2 * cuda.A_int8.shape[1]), dtype=torch.int8, device="cuda")
        _sm100.run_o0(wide[:, : cuda.A_int8.shape[1]], cuda.A_scale, cuda.W_mxfp4, cuda.W_scale, "cold")
    with pytest.raises(RuntimeError, match="K must be divisible by 64"):
        a = torch.zeros((4, 32), dtype=torch.int8, device="cuda")
        _sm100.run_o0(a, torch.ones(4, device="cuda"), torch.zeros((4, 16), dtype=torch.uint8, device="cuda"),
                      torch.zeros((4, 1), dtype=torch.uint8, device="cuda"), "cold")


def test_host_session_matches_device_path(golden_dir):
    from adangel_oyzl_b200.kernels import HostSession

    ref, args = golden_inputs(golden_dir, "fp16_seed2026_132x132x256")
    a_int8, a_scale, w_mx, w_sc = (np.ascontiguousarray(a) for a in args)
    for variant, key in (("o0", "o0_output"), ("o1", "o1_output"), ("o2", "o2_output")):
        session = HostSession(variant, 256, w_mx, w_sc)
        y = np.empty((a_int8.shape[0], w_mx.shape[0]), dtype=np.float32)
        session.run(a_int8, a_scale, y)
        session.run(a_int8, a_scale, y)
        session.close()
        np.testing.assert_allclose(y, ref[key], rtol=1e-3, atol=1e-3)


def test_host_sessions_overlapped_submit_wait(golden_dir):
    # the three variants' passes in flight together (submit all, then wait all), pinned buffers
    import torch
    from adangel_oyzl_b200.kernels import HostSession

    ref, args = golden_inputs(golden_dir, "fp16_seed2026_132x132x256")
    a_int8, a_scale, w_mx, w_sc = (torch.from_numpy(np.ascontiguousarray(a)) for a in args)
    a_pin, s_pin = a_int8.pin_memory(), a_scale.pin_memory()
    sessions = {v: HostSession(v, 256, w_mx, w_sc) for v in ("o0", "o1", "o2")}
    outs = {v: torch.empty((a_int8.shape[0], w_mx.shape[0]), dtype=torch.float32).pin_memory() for v in sessions}
    for _ in range(2):
        for v, s in sessions.items():
            s.submit(a_pin, s_pin, outs[v])
        for s in sessions.values():
            s.wait()
    # a second submit before the wait is refused, and the session stays usable
    sessions["o1"].submit(a_pin, s_pin, outs["o1"])
    with pytest.raises(RuntimeError, match="already has a pass in flight"):
        sessions["o1"].submit(a_pin, s_pin, outs["o1"])
    sessions["o1"].wait()
    for s in sessions.values():
        s.close()
    np.testing.assert_allclose(outs["o0"].numpy(), ref["o0_output"], rtol=1e-3, atol=1e-3)
    np.testing.assert_array_equal(outs["o1"].numpy(), ref["o1_output"])
    np.testing.assert_allclose(outs["o2"].numpy(), ref["o2_output"], rtol=1e-3, atol=1e-3)


def test_o1_host_session_operand_paths(golden_dir):
    # an O1 session runs on BF16 operands (weight scale folded into W) and must fall back to the INT8
    # operands, with the oracle's bits, when a weight scale code or an activation scale leaves that
    # kernel's exact range, and for decode-sized M
    from adangel_oyzl_b200.kernels import HostSession
    from oracle import adangel_oracle as orc

    a_int8, a_scale, w_mx, w_sc = (np.ascontiguousarray(a) for a in orc.canonical_inputs(160, 256, 256, seed=41))
    want = orc.run_o1(a_int8, a_scale, w_mx, w_sc)["output"]
    y = np.empty((160, 256), dtype=np.float32)
    session = HostSession("o1", 256, w_mx, w_sc)
    np.testing.assert_array_equal(session.run(a_int8, a_scale, y), want)            # BF16 operands
    y40 = np.empty((40, 256), dtype=np.float32)
    np.testing.assert_array_equal(session.run(a_int8[:40], a_scale[:40], y40), want[:40])  # decode kernel
    odd_scale = a_scale.copy()
    odd_scale[7] = np.float32(2.0 ** -50)                                               # outside [2^-46, 2^30]
    want_odd = orc.run_o1(a_int8, odd_scale, w_mx, w_sc)["output"]
    np.testing.assert_array_equal(session.run(a_int8, odd_scale, y), want_odd)        # refused, INT8 fallback
    np.testing.assert_array_equal(session.run(a_int8, a_scale, y), want)              # and back
    session.close()
    odd_w = w_sc.copy()
    odd_w[3, 2] = 230                                                                   # outside [48, 208]
    want_w = orc.run_o1(a_int8, a_scale, w_mx, odd_w)["output"]
    session = HostSession("o1", 256, w_mx, odd_w)
    np.testing.assert_array_equal(session.run(a_int8, a_scale, y), want_w)
    session.close()


def test_harness_o1_operand_paths():
    # the timing harness runs O1 on BF16 operands while the scales are inside that kernel's exact range and on
    # the reference's INT8 operands otherwise; both give the oracle's bits and the INT8 form of W is returned
    import torch

    from adangel_oyzl_b200.ops import _sm100

    a_int8, a_scale, w_mx, w_sc = (np.ascontiguousarray(a) for a in orc.canonical_inputs(192, 256, 256, seed=43))
    for odd in (False, True):
        sc = w_sc.copy()
        if odd:
            sc[9, 1] = 231
        dev = [torch.from_numpy(x).cuda() for x in (a_int8, a_scale, w_mx, sc)]
        result = _sm100.benchmark("o1", "steady_state", *dev, 1, 2)
        want = orc.run_o1(a_int8, a_scale, w_mx, sc)
        assert result["kernel"]["kernel_symbol"] == ("gemm_o1_kernel" if odd else "gemm_o1_bf16_kernel")
        assert "activation_conversion" not in result["timings_ms"]
        split = _sm100.benchmark("o1", "steady_state", *dev, 1, 2, o1_split_activation_stage=True)
        assert ("activation_conversion" in split["timings_ms"]) == (not odd)
        np.testing.assert_array_equal(split["output"].cpu().numpy(), want["output"])
        np.testing.assert_array_equal(result["output"].cpu().numpy(), want["output"])
        np.testing.assert_array_equal(result["converted_weight"].cpu().numpy(), orc.mxfp4_to_int8_base(w_mx))
