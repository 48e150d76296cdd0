"""CPU tests: the C-ABI library loads and exports every declared symbol; host-side logic of the
package (schema, dispatch, metrics, synthetic generator, partitioning) behaves like the reference."""

import re
from pathlib import Path

import numpy as np
import pytest

from oracle import adangel_oracle as orc

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_declared_symbols():
    from adangel_oyzl_b200.ops import _sm100

    header = (ROOT / "include" / "adangel_b200.h").read_text()
    declared = set(re.findall(r"\b(adg_[a-z0-9_]+)\s*\(", header))
    declared -= {"adg_bench_args", "adg_session"}
    assert declared, "no declarations found"
    lib = _sm100.library()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(_sm100.EXPORTED_SYMBOLS)
    assert lib.adg_abi_version() == 104
    caps = _sm100.capabilities()
    for key in ("compiled_sm100a", "o0_fp16_tc", "o1_int8_tc", "o2_mxf4_block_scale", "o2_cutlass_tiled"):
        assert caps[key] is True
    assert lib.adg_o2_tiled_scale_bytes(4096, 4096) == 4096 * 128
    assert lib.adg_o2_tiled_scale_bytes(132, 320) == 256 * 16


def test_no_cpu_fallback_without_gpu():
    import torch

    from adangel_oyzl_b200.ops import run_o0
    from adangel_oyzl_b200.ops.extension import native_status, require_native
    from adangel_oyzl_b200.synthetic import canonical_inputs

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    status = native_status()
    assert not status.available and status.reason == "CUDA is not available"
    with pytest.raises(RuntimeError, match="formal SM100 backend unavailable"):
        require_native()
    inputs = canonical_inputs(64, 64, 64)
    with pytest.raises(RuntimeError, match="CUDA is not available"):
        run_o0(inputs)
    with pytest.raises(ValueError, match="unknown backend"):
        run_o0(inputs, backend="reference")
    with pytest.raises(ValueError, match="unknown timing mode"):
        run_o0(inputs, mode="warm")


def test_validate_prepared_contract():
    import torch

    from adangel_oyzl_b200.schema import PreparedInputs, validate_prepared
    from adangel_oyzl_b200.synthetic import canonical_inputs

    good = canonical_inputs(64, 32, 128)
    validate_prepared(good)
    assert good.shape == (64, 32, 128)
    with pytest.raises(ValueError, match="formal experiment requires 4096"):
        validate_prepared(good, formal=True)
    bad = PreparedInputs("x", good.A_int8, good.A_scale, good.W_mxfp4, good.W_scale.clone().fill_(255))
    with pytest.raises(ValueError, match="UE8M0 NaN"):
        validate_prepared(bad)
    with pytest.raises(ValueError, match="A_scale"):
        validate_prepared(PreparedInputs("x", good.A_int8, good.A_scale.double(), good.W_mxfp4, good.W_scale))
    with pytest.raises(ValueError, match="K must be divisible by 64"):
        validate_prepared(PreparedInputs("x", torch.zeros((4, 32), dtype=torch.int8), torch.ones(4),
                                         torch.zeros((4, 16), dtype=torch.uint8), torch.zeros((4, 1), dtype=torch.uint8)))
    with pytest.raises(TypeError):
        validate_prepared(PreparedInputs("x", good.A_int8.numpy(), good.A_scale, good.W_mxfp4, good.W_scale))


@pytest.mark.parametrize("shape", [(64, 48, 128), (256, 512, 1024)])
def test_synthetic_generator_matches_oracle(shape):
    from adangel_oyzl_b200.synthetic import canonical_inputs

    p = canonical_inputs(*shape)
    want = orc.canonical_inputs(*shape)
    for got, ref in zip((p.A_int8, p.A_scale, p.W_mxfp4, p.W_scale), want):
        np.testing.assert_array_equal(got.numpy(), ref)


def test_synthetic_quantizer_edge_blocks():
    import torch

    from adangel_oyzl_b200.synthetic import quantize_mxfp4

    rows = [np.zeros(32), np.full(32, 6.0), np.where(np.arange(32) % 2, 6.0, -6.0), np.full(32, 1e-40),
            np.full(32, 1e30), np.random.default_rng(9).uniform(-10, 10, 32), np.full(32, -1e-3)]
    x = np.stack(rows).astype(np.float32)
    packed, scales = quantize_mxfp4(torch.from_numpy(x))
    want_packed, want_scales = orc.quantize_mxfp4(x)
    np.testing.assert_array_equal(packed.numpy(), want_packed)
    np.testing.assert_array_equal(scales.numpy(), want_scales)


def test_metrics_match_reference_definitions():
    # reference tests/unit/test_metrics.py
    from adangel_oyzl_b200.benchmark import percentile, summarize_samples

    s = summarize_samples([1, 2, 3, 4])
    assert s["median_ms"] == 2.5 and s["iqr_ms"] == 1.5 and s["count"] == 4
    assert percentile([0, 10], 25) == 2.5
    with pytest.raises(ValueError):
        summarize_samples([])


def test_kernel_and_timing_metadata():
    from adangel_oyzl_b200.ops import _sm100

    for mode in ("conversion_only", "compute_only", "cold", "steady_state"):
        meta = _sm100._timing_metadata(mode, 100)
        assert meta["strategy"] == "conversion_amortized_end_to_end_direct"
        assert meta["conversion_stage_timing"] == "isolated_batched_cuda_event_average"
        assert meta["mode_total_inner_repeats"] == (100 if mode == "conversion_only" else 1)
    assert "kind::f16" in _sm100.kernel_metadata("o0", 4096, 4096, 4096)["mma_family"]
    assert "kind::i8" in _sm100.kernel_metadata("o1", 4096, 4096, 4096)["mma_family"]
    assert "kind::mxf4.block_scale" in _sm100.kernel_metadata("o2", 4096, 4096, 4096)["mma_family"]
    assert "kind::i8" in _sm100.kernel_metadata("o1x", 4096, 4096, 4096)["mma_family"]


def test_plan_info_follows_the_planner():
    # the library's own account of what it would launch (adg_plan_info; 148 SMs assumed without a device)
    from adangel_oyzl_b200.ops import _sm100

    big = _sm100.plan_info("o2", 16384, 3584, 8192)
    assert big["kernel_symbol"] == "gemm_pair_kernel<2>" and big["tile"] == [256, 256] and big["cluster"] == [2, 1, 1]
    assert _sm100.plan_info("o2", 16384, 3584, 8192, fused=True)["kernel_symbol"] == "gemm_pair_kernel<2,fused>"
    assert _sm100.plan_info("o2", 4096, 4096, 4096)["kernel_symbol"] == "gemm_acc_kernel<2>"
    assert _sm100.plan_info("o0", 4096, 4096, 4096)["kernel_symbol"] == "gemm_pair_kernel<0>"
    fused = _sm100.plan_info("o0", 4096, 4096, 4096, fused=True)
    assert fused["fused_activation_conversion"] and fused["threads"] == 512
    assert _sm100.plan_info("o0", 2048, 128, 4096)["tile"] == [128, 128]
    assert _sm100.plan_info("o1", 4096, 4096, 4096)["kernel_symbol"] == "gemm_o1_kernel"
    assert _sm100.plan_info("o1", 4096, 4096, 4096, o1_bf16=True)["kernel_symbol"] == "gemm_o1_bf16_kernel"
    assert _sm100.plan_info("o1", 16, 4096, 4096, o1_bf16=True)["kernel_symbol"] == "gemm_o1_decode_kernel"
    assert _sm100.plan_info("o1", 16, 11008, 4096, o1_bf16=True)["kernel_symbol"] == "gemm_o1_skinny_kernel"
    assert _sm100.plan_info("o1", 8, 11008, 4096, o1_bf16=True)["threads"] == 128
    assert _sm100.plan_info("o1", 64, 4096, 4096, o1_bf16=True)["kernel_symbol"] == "gemm_o1_skinny_kernel"
    assert _sm100.plan_info("o2", 64, 4096, 4096, fused=True)["kernel_symbol"] == "gemm_o2_skinny_kernel"
    assert _sm100.plan_info("o1x", 4096, 4096, 4096)["mma_shape"] == [128, 256, 32]
    with pytest.raises(RuntimeError, match="K must be divisible by 64"):
        _sm100.plan_info("o0", 128, 128, 96)


def test_sources_issue_blackwell_instructions():
    # the sm_100a analogue of the reference's static source contract (tests/unit/test_project_contract.py)
    csrc = ROOT / "adangel_oyzl_b200" / "csrc"
    common = (csrc / "common.cuh").read_text()
    for token in ("tcgen05.mma.cta_group::1.kind::f16", "tcgen05.mma.cta_group::1.kind::i8",
                  "tcgen05.mma.cta_group::1.kind::mxf4.block_scale", "cp.async.bulk.tensor.2d.shared::cluster.global",
                  "tcgen05.alloc", "tcgen05.ld.sync.aligned.32x32b", "tcgen05.cp.cta_group::1.32x128b.warpx4",
                  "mbarrier.try_wait.parity"):
        assert token in common, token
    text = "".join(p.read_text() for p in csrc.iterdir() if p.suffix in (".cu", ".cuh", ".h"))
    # no library GEMMs and no Hopper-only MMA
    for forbidden in ("cublas", "cutlass/", "cute/", "wgmma"):
        assert forbidden not in text, forbidden
    assert "compute_100a" in (ROOT / "adangel_oyzl_b200" / "build.py").read_text()


def test_shard_ranges_cover_exactly():
    from adangel_oyzl_b200.parallel import all_ranges, shard_range

    for n in (28672, 4096, 11008, 132, 100, 128):
        for world in (1, 2, 4, 8):
            ranges = all_ranges(n, world)
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(r0 % 128 == 0 or r0 == n for r0, _ in ranges)
            sizes = [r1 - r0 for r0, r1 in ranges]
            assert max(sizes) - min(sizes) <= 128 + 127
    assert shard_range(28672, 8, 3) == (3 * 3584, 4 * 3584)
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def test_instruction_audit_passes(tmp_path):
    # the counterpart of the reference's scripts/audit_instructions.sh: every production kernel's PTX
    # (compiled from this project's sources) holds its TMA / tensor-core instruction family
    import shutil

    if shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists():
        pytest.skip("nvcc not available")
    from adangel_oyzl_b200.audit import audit

    result = audit(tmp_path)
    assert result["status"] == "PASS", result["lines"]
    assert (tmp_path / "summary.txt").read_text().startswith("status=PASS")
    assert result["kernels"] >= 12


def test_c_abi_rejects_misaligned_and_null_pointers():
    # the conversion kernels use 16-byte vector accesses (4-byte for scale arrays and flag words): a pointer
    # that would fault on the device is refused on the host, before any CUDA call
    from adangel_oyzl_b200.ops import _sm100

    lib = _sm100.library()
    base = 0x7F0000000000  # never dereferenced: every call below must fail in its argument checks
    cases = [
        (lib.adg_int8_to_fp16, (base + 1, base, base, 64, 64, None), "A_int8 must be 16-byte aligned"),
        (lib.adg_int8_to_fp16, (base, base + 2, base, 64, 64, None), "A_scale must be 4-byte aligned"),
        (lib.adg_int8_to_fp16, (base, base, base + 8, 64, 64, None), "out_fp16 must be 16-byte aligned"),
        (lib.adg_mxfp4_to_fp16, (base + 4, base, base, 64, 64, None), "W_mxfp4 must be 16-byte aligned"),
        (lib.adg_mxfp4_to_fp16, (base, None, base, 64, 64, None), "W_scale must not be NULL"),
        (lib.adg_mxfp4_to_int8, (base, base + 3, 64, 64, None), "out_int8 must be 16-byte aligned"),
        (lib.adg_mxfp4_to_bf16_scaled, (base, base, base, base + 2, 64, 64, None), "range_flag must be 4-byte aligned"),
        (lib.adg_int8_to_bf16, (base, base, base + 1, base, 64, 64, None), "out_bf16 must be 16-byte aligned"),
        (lib.adg_o2_quantize_activation, (base, base, base + 8, None, base, 64, 64, None), "A_mxfp4 must be 16-byte aligned"),
        (lib.adg_o2_quantize_activation, (base, base, base, base + 1, base, 64, 64, None), "sf_natural must be 4-byte aligned"),
        (lib.adg_o2_quantize_activation, (base, base, base, None, None, 64, 64, None), "sf_tiled must not be NULL"),
        (lib.adg_o2_tile_scales, (base, base + 4, 64, 64, None), "sf_tiled must be 16-byte aligned"),
        (lib.adg_quantize_int8_per_row, (base + 4, 0, base, base, 64, 64, None), "x must be 16-byte aligned"),
        (lib.adg_quantize_mxfp4, (base, 0, base + 1, base, 64, 64, None), "packed must be 16-byte aligned"),
        (lib.adg_o1x_prepare_weight, (base, base, base + 1, base, base, 64, 64, None), "must be 16-byte aligned"),
        (lib.adg_int8_to_fp16, (base, base, base, 64, 96, None), "K must be divisible by 64"),
    ]
    for fn, args, message in cases:
        assert fn(*args) != 0, message
        assert message in lib.adg_last_error().decode(), (message, lib.adg_last_error())
    # the gather over peer memory: block geometry is checked before any CUDA call
    import ctypes

    def blocks(src, col0, width, count=1):
        b = _sm100.PeerBlocks()
        b.src[0], b.col0[0], b.width[0], b.count = src, col0, width, count
        return ctypes.byref(b)

    gather_cases = [
        ((blocks(base, 0, 64), base + 4, 8, 128, None), "y must be 16-byte aligned"),
        ((blocks(base, 0, 64), base, 8, 126, None), "ldy a multiple of 4"),
        ((blocks(base + 8, 0, 64), base, 8, 128, None), "block pointers must be non-NULL and 16-byte aligned"),
        ((blocks(base, 2, 64), base, 8, 128, None), "block columns must be multiples of 4"),
        ((blocks(base, 96, 64), base, 8, 128, None), "inside the row"),
        ((blocks(base, 0, 64, count=0), base, 8, 128, None), "bad block count"),
    ]
    for args, message in gather_cases:
        assert lib.adg_gather_columns_pull(*args) != 0, message
        assert message in lib.adg_last_error().decode(), (message, lib.adg_last_error())
