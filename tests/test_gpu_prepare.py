"""The sample-preparation quantizers (CUDA) against the CPU oracle, bit for bit, and the prepared
directory they feed.  Inputs include the cases the reference's codec tests pin: ties on the E2M1
grid, saturation, negative values that round to zero (code 8) and -0.0 (code 0), all-zero rows and
blocks, subnormal and huge magnitudes, block maxima just below a power of two (where an FP32
floor(log2) would be off by one) and FP16 sources."""

import numpy as np
import pytest

from oracle import adangel_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from adangel_oyzl_b200 import kernels

    return kernels


def _special_matrix(rows, k, rng):
    x = rng.standard_normal((rows, k)).astype(np.float32)
    x[:, rng.choice(k, max(1, k // 200), replace=False)] *= 20.0
    grid = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 0.1, 0.0], dtype=np.float32)
    # rows of exact ties / grid points at several block exponents, both signs
    for r, e in enumerate((-20, -3, 0, 2, 9)):
        vals = np.tile(np.concatenate([grid, -grid]), k // 34 + 1)[:k] * np.float32(2.0 ** e)
        x[r] = vals
        x[r, ::32] = np.float32(6.0 * 2.0 ** e)  # fixes every block's amax: exponent e for all blocks
    x[5] = 0.0                              # all-zero row
    x[6, :64] = 0.0                         # all-zero blocks inside a row
    x[7, :32] = -0.0
    x[8] = rng.standard_normal(k).astype(np.float32) * np.float32(1e-42)   # subnormal
    x[9] = rng.standard_normal(k).astype(np.float32) * np.float32(1e36)    # near the top of FP32
    # block maxima a few ulps below powers of two
    for b, e in enumerate(range(-12, 12)):
        if (b + 1) * 32 > k:
            break
        blk = rng.uniform(-0.5, 0.5, 32).astype(np.float32) * np.float32(2.0 ** e)
        blk[3] = np.nextafter(np.float32(2.0 ** e), np.float32(0), dtype=np.float32) if b % 2 else -np.nextafter(
            np.nextafter(np.float32(2.0 ** e), np.float32(0), dtype=np.float32), np.float32(0), dtype=np.float32)
        x[10, b * 32:(b + 1) * 32] = blk
    x[11, 5] = -1e-30  # a small negative next to large values: rounds to zero, keeps its sign bit
    return x


@pytest.mark.parametrize("dtype", ["float32", "float16"])
@pytest.mark.parametrize("shape", [(16, 64), (40, 1024), (300, 4096)])
def test_quantizers_match_oracle(K, shape, dtype):
    import torch

    rng = np.random.default_rng(1234 + shape[1])
    x = _special_matrix(*shape, rng) if shape[0] >= 16 else rng.standard_normal(shape).astype(np.float32)
    if dtype == "float16":
        with np.errstate(over="ignore"):
            x = x.astype(np.float16)
        x[~np.isfinite(x)] = 0
    dx = torch.from_numpy(x).cuda()
    x32 = x.astype(np.float32)
    q, s = K.quantize_int8_per_row(dx)
    oq, os_ = orc.quantize_int8_per_row(x32)
    np.testing.assert_array_equal(s.cpu().numpy(), os_)
    np.testing.assert_array_equal(q.cpu().numpy(), oq)
    packed, codes = K.quantize_mxfp4(dx)
    opacked, ocodes = orc.quantize_mxfp4(x32)
    np.testing.assert_array_equal(codes.cpu().numpy(), ocodes)
    np.testing.assert_array_equal(packed.cpu().numpy(), opacked)


def test_quantizers_reject_bad_input(K):
    import torch

    x = torch.zeros((4, 64), device="cuda")
    x[1, 3] = float("nan")
    with pytest.raises(ValueError, match="activation contains NaN/Inf"):
        K.quantize_int8_per_row(x)
    with pytest.raises(ValueError, match="MXFP4 input contains NaN/Inf"):
        K.quantize_mxfp4(x)
    with pytest.raises(ValueError, match="divisible by 32"):
        K.quantize_mxfp4(torch.zeros((4, 48), device="cuda"))
    with pytest.raises(RuntimeError, match="float32 or float16"):
        K.quantize_int8_per_row(torch.zeros((4, 64), device="cuda", dtype=torch.float64))


def test_canonical_sample_on_gpu_equals_cpu_generator(K):
    # the prepared sample made by the kernels is the one the (torch, CPU) generator makes
    import torch
    from adangel_oyzl_b200 import synthetic
    from adangel_oyzl_b200.trace.prepare import quantize_sample

    a, w = synthetic.canonical_floats(256, 384, 1024, seed=77)
    cpu = synthetic.canonical_inputs(256, 384, 1024, seed=77)
    gpu = quantize_sample("s", a, w)
    for name in ("A_int8", "A_scale", "W_mxfp4", "W_scale"):
        assert torch.equal(getattr(gpu, name).cpu(), getattr(cpu, name)), name


def test_prepare_synthetic_directory_feeds_the_ops(K, tmp_path):
    import torch
    from adangel_oyzl_b200.trace import storage
    from adangel_oyzl_b200.trace.prepare import prepare_synthetic

    records = prepare_synthetic([(128, 128, 256), (40, 136, 64)], tmp_path / "prepared", seed=3)
    manifest = storage.load_manifest(tmp_path / "prepared")
    assert [r["sample_id"] for r in manifest["samples"]] == [r["sample_id"] for r in records]
    for record in manifest["samples"]:
        sample = storage.load_prepared(tmp_path / "prepared" / record["file"], device="cuda", expected_sha256=record["sha256"])
        y1 = K.gemm_o1(sample.A_int8, sample.A_scale, K.mxfp4_to_int8(sample.W_mxfp4), sample.W_scale)
        K.check_status()
        want = orc.run_o1(sample.A_int8.cpu().numpy(), sample.A_scale.cpu().numpy(), sample.W_mxfp4.cpu().numpy(),
                          sample.W_scale.cpu().numpy())["output"]
        np.testing.assert_array_equal(y1.cpu().numpy(), want)
    with pytest.raises(FileExistsError):
        prepare_synthetic([(128, 128, 256)], tmp_path / "prepared")
