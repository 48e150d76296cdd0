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


def test_no_alloc_async_status_is_reported_and_cleared():
    """An asynchronous call (synchronize=0) leaves its kernels' status words inside the built-in array; the
    status query and adg_check_status must both find, report and clear a non-zero word there.  The word is
    planted from the host with a copy -- no kernel is made to give up."""
    import ctypes

    import torch

    from adangel_oyzl_b200 import kernels as K

    m, n, k = 128, 256, 256
    a_int8, a_scale, w_mx, w_sc = orc.canonical_inputs(m, n, k, seed=103)
    da, ds, dw, dws = (torch.from_numpy(x).cuda() for x in (a_int8, a_scale, w_mx, w_sc))
    w_tiled = K.o2_tile_scales(dws)
    out = torch.empty((m, n), device="cuda")
    K.o2_linear_noalloc(da, ds, dw, w_tiled, out, synchronize=False)
    K.o2_linear_noalloc_status()  # healthy: nothing to report
    np.testing.assert_allclose(out.cpu().numpy(), orc.run_o2(a_int8, a_scale, w_mx, w_sc)["output"], rtol=RTOL, atol=ATOL)

    lib = K._lib()
    addr, size = ctypes.c_void_p(), ctypes.c_int()
    assert lib.adg_o2_linear_noalloc_status_words(ctypes.byref(addr), ctypes.byref(size)) == 0
    assert size.value >= 16
    from cuda.bindings import runtime as cudart  # cuda-python: the same primary context as the library's runtime

    words = torch.tensor([1, 0x123, 7, 0], dtype=torch.int32)  # code 1 = a wait that gave up, tag, block
    for check in (K.o2_linear_noalloc_status, K.check_status):
        (err,) = cudart.cudaMemcpy(addr.value, words.data_ptr(), 16, cudart.cudaMemcpyKind.cudaMemcpyHostToDevice)
        assert int(err) == 0
        with pytest.raises(RuntimeError, match="adg_o2_linear_noalloc: kernel wait timeout: code=1"):
            check()
        check()  # reported once, then clear
