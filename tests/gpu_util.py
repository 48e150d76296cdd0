"""Helpers shared by the GPU parity tests."""

import numpy as np


def to_cuda(*arrays):
    import torch

    return tuple(torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays)


def golden_inputs(golden_dir, name):
    ref = np.load(golden_dir / f"{name}.npz")
    return ref, (ref["A_int8"], ref["A_scale"], ref["W_mxfp4"], ref["W_scale"])


def assert_requant_matches(codes, scales, a_int8, a_scale, orc):
    """Bit-exact comparison of re-quantized activation codes/scales with the oracle.

    A block may differ only in the documented way: the block maximum lies within 8 ulps below a
    power of two, where the FP32-log2 form of the reference's tensor quantizer picks an exponent
    one larger than the exact one that its scalar helper and CUDA kernel (and this build) use.
    The oracle used here is the exact form, so the expected number of differing blocks is zero.
    """
    act = orc.dequantize_int8_per_row(a_int8, a_scale, np.float32)
    want_codes, want_scales = orc.quantize_mxfp4(act)
    np.testing.assert_array_equal(scales, want_scales)
    np.testing.assert_array_equal(codes, want_codes)
