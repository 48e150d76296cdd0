"""B200 (sm_100a) backend for ADAngel's O0/O1/O2 quantized GEMMs ``Y = A @ W.T``.

The package mirrors the reference project's Python surface for this path — the ``ops`` loader,
capability gate and unified O0/O1/O2 dispatch, ``python -m adangel_oyzl_b200 doctor
--require-native`` and the benchmark record schema — on top of a C-ABI shared library of
hand-written CUDA kernels (``include/adangel_b200.h``).  There is no CPU fallback.
"""

__version__ = "0.1.0"
