"""The allocation-free O2 entry point must give the same result as the regular O2 path.

Some users of the library cannot allocate device memory when they call it: an inference server
whose own pool already holds all of the GPU's memory, or a decode loop that may not pay for the
device-wide synchronisation of cudaMalloc.  ``adg_o2_linear_noalloc`` serves them from a fixed
scratch array inside the library.  This test calls it through the C ABI twice in a row, with a
larger and then a smaller activation so that leftovers of the first call are in the shared array
when the second runs, and compares each result with the regular entry points
(``adg_o2_quantize_activation`` + ``adg_gemm_o2``) and with the CPU oracle.
"""

import numpy as np
import pytest

from oracle import adangel_oracle as orc

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-3  # the tolerance of the other O2 output tests


def test_no_alloc_matches_regular_path_on_two_calls():
    import torch

    from adangel_oyzl_b200 import kernels as K

    n, k1 = 384, 1024
    for call, (m, k) in enumerate(((300, k1), (64, 256))):
        a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(m, n, k, seed=100 + call)
        da, ds, dw, dws = (torch.from_numpy(x).cuda() for x in (a_int8, a_scale, w_mx, w_sc))
        w_tiled = K.o2_tile_scales(dws)
        out = torch.full((m, n), float("nan"), device="cuda")
        K.o2_linear_noalloc(da, ds, dw, w_tiled, out)  # synchronises and reports kernel errors itself
        codes, _, sfa = K.o2_quantize_activation(da, ds)
        ref = K.gemm_o2(codes, sfa, dw, w_tiled)
        K.check_status()
        got = out.cpu().numpy()
        np.testing.assert_allclose(got, ref.cpu().numpy(), rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(got, orc.run_o2(a_int8, a_scale, w_mx, w_sc)["output"], rtol=RTOL, atol=ATOL)


def test_no_alloc_rejects_oversized_activation():
    import torch

    from adangel_oyzl_b200 import kernels as K

    m, n, k = 4096, 128, 4096  # 8 MiB of codes: beyond the 4 MiB scratch
    da = torch.zeros((m, k), dtype=torch.int8, device="cuda")
    ds = torch.ones((m,), dtype=torch.float32, device="cuda")
    dw = torch.zeros((n, k // 2), dtype=torch.uint8, device="cuda")
    w_tiled = torch.zeros((K.tiled_scale_bytes(n, k),), dtype=torch.uint8, device="cuda")
    out = torch.empty((m, n), device="cuda")
    with pytest.raises(RuntimeError, match="too large for the built-in scratch"):
        K.o2_linear_noalloc(da, ds, dw, w_tiled, out)
