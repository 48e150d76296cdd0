"""Tensor-level wrappers of the individual C-ABI kernels (conversions and GEMMs).

Each function validates shapes/dtypes, allocates the output on the inputs' device, enqueues the
kernel on torch's current stream and returns the output tensor(s) without synchronising.  These are
the building blocks behind :mod:`adangel_oyzl_b200.ops` and the N-sharded multi-GPU driver.
"""

from __future__ import annotations

import ctypes

from .ops import _sm100


def _stream(t):
    import torch

    return torch.cuda.current_stream(t.device).cuda_stream


def _lib():
    return _sm100.library()


def _require(cond, message):
    if not cond:
        raise RuntimeError(message)


def mxfp4_to_fp16(w_mxfp4, w_scale):
    import torch

    n, kh = w_mxfp4.shape
    k = kh * 2
    _require(w_mxfp4.is_cuda and w_mxfp4.dtype == torch.uint8 and w_mxfp4.is_contiguous(), "W_mxfp4 must be contiguous CUDA uint8")
    _require(w_scale.dtype == torch.uint8 and tuple(w_scale.shape) == (n, k // 32) and w_scale.is_contiguous(), "invalid W_scale")
    out = torch.empty((n, k), dtype=torch.float16, device=w_mxfp4.device)
    with torch.cuda.device(w_mxfp4.device):
        _sm100._check(_lib().adg_mxfp4_to_fp16(w_mxfp4.data_ptr(), w_scale.data_ptr(), out.data_ptr(), n, k, _stream(out)))
    return out


def torch_device(device):
    import torch

    return torch.cuda.device(device)


def int8_to_fp16(a_int8, a_scale):
    import torch

    m, k = a_int8.shape
    _require(a_int8.is_cuda and a_int8.dtype == torch.int8 and a_int8.is_contiguous(), "A_int8 must be contiguous CUDA int8")
    _require(a_scale.dtype == torch.float32 and tuple(a_scale.shape) == (m,), "invalid A_scale")
    out = torch.empty((m, k), dtype=torch.float16, device=a_int8.device)
    with torch.cuda.device(a_int8.device):
        _sm100._check(_lib().adg_int8_to_fp16(a_int8.data_ptr(), a_scale.data_ptr(), out.data_ptr(), m, k, _stream(out)))
    return out


def mxfp4_to_int8(w_mxfp4):
    import torch

    n, kh = w_mxfp4.shape
    _require(w_mxfp4.is_cuda and w_mxfp4.dtype == torch.uint8 and w_mxfp4.is_contiguous(), "W_mxfp4 must be contiguous CUDA uint8")
    out = torch.empty((n, kh * 2), dtype=torch.int8, device=w_mxfp4.device)
    with torch.cuda.device(w_mxfp4.device):
        _sm100._check(_lib().adg_mxfp4_to_int8(w_mxfp4.data_ptr(), out.data_ptr(), n, kh * 2, _stream(out)))
    return out


def new_range_flag(device):
    """The zeroed device word that the BF16-operand O1 conversions and GEMM share."""
    import torch

    return torch.zeros(1, dtype=torch.int32, device=device)


def mxfp4_to_bf16_scaled(w_mxfp4, w_scale, range_flag):
    """W as BF16 of e2m1 * 2^(scale-127) (exact): the weight operand of :func:`gemm_o1_bf16`."""
    import torch

    n, kh = w_mxfp4.shape
    _require(w_mxfp4.is_cuda and w_mxfp4.dtype == torch.uint8 and w_mxfp4.is_contiguous(), "W_mxfp4 must be contiguous CUDA uint8")
    _require(w_scale.dtype == torch.uint8 and tuple(w_scale.shape) == (n, kh * 2 // 32) and w_scale.is_contiguous(), "invalid W_scale")
    out = torch.empty((n, kh * 2), dtype=torch.bfloat16, device=w_mxfp4.device)
    with torch.cuda.device(w_mxfp4.device):
        _sm100._check(_lib().adg_mxfp4_to_bf16_scaled(
            w_mxfp4.data_ptr(), w_scale.data_ptr(), out.data_ptr(), range_flag.data_ptr(), n, kh * 2, _stream(out)))
    return out


def int8_to_bf16(a_int8, a_scale, range_flag):
    """A's integers as BF16 (exact): the activation operand of :func:`gemm_o1_bf16`."""
    import torch

    m, k = a_int8.shape
    _require(a_int8.is_cuda and a_int8.dtype == torch.int8 and a_int8.is_contiguous(), "A_int8 must be contiguous CUDA int8")
    _require(a_scale.dtype == torch.float32 and tuple(a_scale.shape) == (m,), "invalid A_scale")
    out = torch.empty((m, k), dtype=torch.bfloat16, device=a_int8.device)
    with torch.cuda.device(a_int8.device):
        _sm100._check(_lib().adg_int8_to_bf16(
            a_int8.data_ptr(), a_scale.data_ptr(), out.data_ptr(), range_flag.data_ptr(), m, k, _stream(out)))
    return out


def tiled_scale_bytes(rows: int, k: int) -> int:
    return int(_lib().adg_o2_tiled_scale_bytes(rows, k))


def o2_quantize_activation(a_int8, a_scale, want_natural=True):
    """Returns (codes [M,K/2] u8, natural scales [M,K/32] u8 or None, tiled scales u8)."""
    import torch

    m, k = a_int8.shape
    _require(a_int8.is_cuda and a_int8.dtype == torch.int8 and a_int8.is_contiguous(), "A_int8 must be contiguous CUDA int8")
    _require(a_scale.dtype == torch.float32 and tuple(a_scale.shape) == (m,), "invalid A_scale")
    dev = a_int8.device
    codes = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
    natural = torch.empty((m, k // 32), dtype=torch.uint8, device=dev) if want_natural else None
    tiled = torch.zeros((tiled_scale_bytes(m, k),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _sm100._check(_lib().adg_o2_quantize_activation(
            a_int8.data_ptr(), a_scale.data_ptr(), codes.data_ptr(),
            natural.data_ptr() if natural is not None else None, tiled.data_ptr(), m, k, _stream(codes)))
    return codes, natural, tiled


def o2_tile_scales(scales):
    import torch

    rows, groups = scales.shape
    _require(scales.is_cuda and scales.dtype == torch.uint8 and scales.is_contiguous(), "scales must be contiguous CUDA uint8")
    tiled = torch.empty((tiled_scale_bytes(rows, groups * 32),), dtype=torch.uint8, device=scales.device)
    with torch.cuda.device(scales.device):
        _sm100._check(_lib().adg_o2_tile_scales(scales.data_ptr(), tiled.data_ptr(), rows, groups * 32, _stream(tiled)))
    return tiled


def _float_dtype_code(x):
    import torch

    _require(x.is_cuda and x.dim() == 2 and x.is_contiguous(), "expected a contiguous rank-2 CUDA tensor")
    _require(x.dtype in (torch.float32, torch.float16), "expected a float32 or float16 tensor")
    return 0 if x.dtype == torch.float32 else 1


def quantize_int8_per_row(x, check_finite: bool = True):
    """Per-row symmetric INT8 of a float32/float16 CUDA matrix: ``(q int8 [M,K], scale f32 [M])``.

    Same contract as the reference's ``quantize_int8_per_row`` (quantization/int8.py:6-17),
    including its rejection of NaN/Inf (a host-side check there too)."""
    import torch

    code = _float_dtype_code(x)
    rows, k = x.shape
    if check_finite and not bool(torch.isfinite(x).all()):
        raise ValueError("activation contains NaN/Inf")
    q = torch.empty((rows, k), dtype=torch.int8, device=x.device)
    scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _sm100._check(_lib().adg_quantize_int8_per_row(x.data_ptr(), code, q.data_ptr(), scale.data_ptr(), rows, k, _stream(q)))
    return q, scale


def quantize_mxfp4(x, check_finite: bool = True):
    """MXFP4 of a float32/float16 CUDA matrix: ``(packed u8 [N,K/2], scale codes u8 [N,K/32])``.

    Same contract as the reference's ``quantize_mxfp4`` (quantization/mxfp4.py:147-180) with the
    exact block exponent of its scalar helper and CUDA kernel."""
    import torch

    code = _float_dtype_code(x)
    rows, k = x.shape
    if k % 32:
        raise ValueError("x must be rank-2 and K must be divisible by 32")
    if check_finite and not bool(torch.isfinite(x).all()):
        raise ValueError("MXFP4 input contains NaN/Inf")
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _sm100._check(_lib().adg_quantize_mxfp4(x.data_ptr(), code, packed.data_ptr(), scales.data_ptr(), rows, k, _stream(packed)))
    return packed, scales


def _output(out, m, n, device):
    import torch

    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=device)
    _require(out.is_cuda and out.device == device, "the output must live on the operands' device")
    _require(out.dtype == torch.float32 and tuple(out.shape) == (m, n) and out.stride(1) == 1, "invalid output tensor")
    return out, int(out.stride(0))


def _operand(t, name, dtype, shape=None, device=None):
    """dtype / device / contiguity / shape check of one GEMM operand (the library sees only pointers)."""
    _require(t.is_cuda, f"{name} must be a CUDA tensor")
    _require(t.dtype == dtype, f"{name} must be {dtype}")
    _require(t.is_contiguous(), f"{name} must be contiguous")
    if shape is not None:
        _require(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}, found {tuple(t.shape)}")
    if device is not None:
        _require(t.device == device, f"{name} must be on {device}")
    return t


def _tiled(t, name, rows, k, device):
    import torch

    _operand(t, name, torch.uint8, device=device)
    _require(t.numel() >= tiled_scale_bytes(rows, k), f"{name} is shorter than the tiled scale layout of {rows} rows x K = {k}")
    return t


def gemm_o0(a_fp16, w_fp16, out=None):
    import torch

    m, k = a_fp16.shape
    n = w_fp16.shape[0]
    _operand(a_fp16, "A_fp16", torch.float16)
    _operand(w_fp16, "W_fp16", torch.float16, (n, k), a_fp16.device)
    out, ldy = _output(out, m, n, a_fp16.device)

    with torch.cuda.device(a_fp16.device):
        _sm100._check(_lib().adg_gemm_o0(a_fp16.data_ptr(), w_fp16.data_ptr(), out.data_ptr(), m, n, k, ldy, _stream(out)))
    return out


def gemm_o1(a_int8, a_scale, w_int8, w_scale, out=None, dump_partials=False):
    import torch

    m, k = a_int8.shape
    n = w_int8.shape[0]
    dev = a_int8.device
    _operand(a_int8, "A_int8", torch.int8)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _operand(w_int8, "W_int8", torch.int8, (n, k), dev)
    _operand(w_scale, "W_scale", torch.uint8, (n, k // 32), dev)
    out, ldy = _output(out, m, n, a_int8.device)
    partials = torch.empty((m, n, k // 32), dtype=torch.int32, device=a_int8.device) if dump_partials else None
    with torch.cuda.device(a_int8.device):
        _sm100._check(_lib().adg_gemm_o1(
            a_int8.data_ptr(), a_scale.data_ptr(), w_int8.data_ptr(), w_scale.data_ptr(), out.data_ptr(),
            partials.data_ptr() if partials is not None else None, m, n, k, ldy, _stream(out)))
    return (out, partials) if dump_partials else out


def gemm_o1_packed(a_int8, a_scale, w_mxfp4, w_scale, out=None):
    """O1 for decode-sized activations straight from the packed MXFP4 weights (same bits as :func:`gemm_o1`;
    M <= 8, or M <= 16 while N/32 does not exceed the SM count -- other shapes raise)."""
    import torch

    m, k = a_int8.shape
    n = w_mxfp4.shape[0]
    dev = a_int8.device
    _operand(a_int8, "A_int8", torch.int8)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _operand(w_mxfp4, "W_mxfp4", torch.uint8, (n, k // 2), dev)
    _operand(w_scale, "W_scale", torch.uint8, (n, k // 32), dev)
    out, ldy = _output(out, m, n, a_int8.device)
    with torch.cuda.device(a_int8.device):
        _sm100._check(_lib().adg_gemm_o1_packed(
            a_int8.data_ptr(), a_scale.data_ptr(), w_mxfp4.data_ptr(), w_scale.data_ptr(), out.data_ptr(), m, n, k, ldy,
            _stream(out)))
    return out


def gemm_o1_bf16(a_bf16, a_scale, w_bf16, range_flag, out=None):
    """O1 on BF16 operands (same bits as :func:`gemm_o1` while ``range_flag`` stays zero; otherwise the
    kernel refuses and the next status check raises)."""
    import torch

    m, k = a_bf16.shape
    n = w_bf16.shape[0]
    dev = a_bf16.device
    _operand(a_bf16, "A_bf16", torch.bfloat16)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _operand(w_bf16, "W_bf16", torch.bfloat16, (n, k), dev)
    _operand(range_flag, "range_flag", torch.int32, device=dev)
    out, ldy = _output(out, m, n, a_bf16.device)
    with torch_device(a_bf16.device):
        _sm100._check(_lib().adg_gemm_o1_bf16(
            a_bf16.data_ptr(), a_scale.data_ptr(), w_bf16.data_ptr(), out.data_ptr(), range_flag.data_ptr(),
            m, n, k, ldy, _stream(out)))
    return out


class O1Weights:
    """W in both forms O1 can consume, made once: INT8 (every input) and BF16 with the scale folded in
    (the fast kernel), plus the two flag words :func:`o1_linear` needs."""

    def __init__(self, w_mxfp4, w_scale):
        import torch

        self.w_scale = w_scale
        self.w_int8 = mxfp4_to_int8(w_mxfp4)
        self.flags = torch.zeros(2, dtype=torch.int32, device=w_mxfp4.device)
        self.w_bf16 = mxfp4_to_bf16_scaled(w_mxfp4, w_scale, self.flags)
        self._workspace = None

    def workspace(self, m, k):
        import torch

        if self._workspace is None or self._workspace.numel() < m * k:
            self._workspace = torch.empty(m * k, dtype=torch.bfloat16, device=self.w_int8.device)
        return self._workspace


def o1_linear(a_int8, a_scale, weights: O1Weights, out=None):
    """O1 for every input without a host synchronisation: the BF16-operand kernel, and behind it the
    INT8-operand kernel, which runs only if the first one refused (``adg_o1_linear``)."""
    import torch

    m, k = a_int8.shape
    n = weights.w_int8.shape[0]
    dev = a_int8.device
    _operand(a_int8, "A_int8", torch.int8)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _require(tuple(weights.w_int8.shape) == (n, k) and weights.w_int8.device == dev, "weights do not match A")
    out, ldy = _output(out, m, n, a_int8.device)
    ws = weights.workspace(m, k)
    with torch_device(a_int8.device):
        _sm100._check(_lib().adg_o1_linear(
            a_int8.data_ptr(), a_scale.data_ptr(), weights.w_int8.data_ptr(), weights.w_scale.data_ptr(),
            weights.w_bf16.data_ptr(), ws.data_ptr(), weights.flags.data_ptr(), out.data_ptr(), m, n, k, ldy, _stream(out)))
    return out


def gemm_o2(a_mxfp4, a_sf_tiled, w_mxfp4, w_sf_tiled, out=None):
    import torch

    m, kh = a_mxfp4.shape
    n = w_mxfp4.shape[0]
    dev = a_mxfp4.device
    _operand(a_mxfp4, "A_mxfp4", torch.uint8)
    _operand(w_mxfp4, "W_mxfp4", torch.uint8, (n, kh), dev)
    _tiled(a_sf_tiled, "a_sf_tiled", m, kh * 2, dev)
    _tiled(w_sf_tiled, "w_sf_tiled", n, kh * 2, dev)
    out, ldy = _output(out, m, n, a_mxfp4.device)
    with torch.cuda.device(a_mxfp4.device):
        _sm100._check(_lib().adg_gemm_o2(
            a_mxfp4.data_ptr(), a_sf_tiled.data_ptr(), w_mxfp4.data_ptr(), w_sf_tiled.data_ptr(), out.data_ptr(),
            m, n, kh * 2, ldy, _stream(out)))
    return out


def o2_linear_noalloc(a_int8, a_scale, w_mxfp4, w_sf_tiled, out, synchronize=True):
    """O2 for callers that cannot allocate device memory: activation re-quantization and GEMM using
    the library's built-in scratch array (``adg_o2_linear_noalloc``).  ``out`` must be provided by
    the caller; nothing is allocated here or in the library.  Calls share the scratch array, so
    they must not overlap on the GPU."""
    import torch

    m, k = a_int8.shape
    n = w_mxfp4.shape[0]
    dev = a_int8.device
    _operand(a_int8, "A_int8", torch.int8)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _operand(w_mxfp4, "W_mxfp4", torch.uint8, (n, k // 2), dev)
    _tiled(w_sf_tiled, "w_sf_tiled", n, k, dev)
    _require(out is not None and out.is_cuda and out.device == dev and out.dtype == torch.float32
             and tuple(out.shape) == (m, n) and out.stride(1) == 1, "invalid output tensor")
    with torch.cuda.device(a_int8.device):
        _sm100._check(_lib().adg_o2_linear_noalloc(
            a_int8.data_ptr(), a_scale.data_ptr(), w_mxfp4.data_ptr(), w_sf_tiled.data_ptr(), out.data_ptr(),
            m, n, k, int(out.stride(0)), _stream(out), 1 if synchronize else 0))
    return out


def o2_linear_noalloc_status(device=None):
    """Status of earlier ``o2_linear_noalloc(..., synchronize=False)`` calls; allocates nothing."""
    import torch

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _sm100._check(_lib().adg_o2_linear_noalloc_status(torch.cuda.current_stream(dev).cuda_stream))


class FusedWorkspace:
    """Buffers of the steady-state passes :func:`o0_linear` / :func:`o2_linear` for up to ``max_m`` rows of K
    elements: the converted operand, O2's tiled scales and -- with ``fuse=True``, which selects the GEMM kernels
    that convert A themselves -- the row counters (zeroed once here; the kernels leave them zero)."""

    def __init__(self, variant: str, max_m: int, k: int, device, want_natural_scales: bool = False, fuse: bool = False):
        import torch

        _require(variant in ("o0", "o2"), "steady-state passes exist for o0 and o2")
        self.variant, self.max_m, self.k = variant, max_m, k
        self.counters = (torch.zeros((int(_lib().adg_fused_workspace_bytes(max_m)) // 4,), dtype=torch.int32, device=device)
                         if fuse else None)
        if variant == "o0":
            self.operand = torch.empty((max_m, k), dtype=torch.float16, device=device)
            self.sf_tiled = self.sf_natural = None
        else:
            self.operand = torch.empty((max_m, k // 2), dtype=torch.uint8, device=device)
            self.sf_tiled = torch.zeros((tiled_scale_bytes(max_m, k),), dtype=torch.uint8, device=device)
            self.sf_natural = torch.empty((max_m, k // 32), dtype=torch.uint8, device=device) if want_natural_scales else None


def o0_linear(a_int8, a_scale, w_fp16, workspace: FusedWorkspace, out=None):
    """O0 steady-state pass, ``adg_o0_linear``: INT8 -> FP16 conversion and GEMM (inside one kernel when the
    workspace was made with ``fuse=True`` and M > 64)."""
    import torch

    m, k = a_int8.shape
    n = w_fp16.shape[0]
    dev = a_int8.device
    _operand(a_int8, "A_int8", torch.int8)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _operand(w_fp16, "W_fp16", torch.float16, (n, k), dev)
    _require(workspace.variant == "o0" and workspace.k == k and m <= workspace.max_m, "workspace does not fit this call")
    out, ldy = _output(out, m, n, dev)
    with torch.cuda.device(dev):
        _sm100._check(_lib().adg_o0_linear(a_int8.data_ptr(), a_scale.data_ptr(), w_fp16.data_ptr(), workspace.operand.data_ptr(),
                                           workspace.counters.data_ptr() if workspace.counters is not None else None,
                                           out.data_ptr(), m, n, k, ldy, _stream(out)))
    return out


def o2_linear(a_int8, a_scale, w_mxfp4, w_sf_tiled, workspace: FusedWorkspace, out=None):
    """O2 steady-state pass, ``adg_o2_linear``: re-quantization and GEMM (inside one kernel when the workspace
    was made with ``fuse=True`` and M > 64)."""
    import torch

    m, k = a_int8.shape
    n = w_mxfp4.shape[0]
    dev = a_int8.device
    _operand(a_int8, "A_int8", torch.int8)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _operand(w_mxfp4, "W_mxfp4", torch.uint8, (n, k // 2), dev)
    _tiled(w_sf_tiled, "w_sf_tiled", n, k, dev)
    _require(workspace.variant == "o2" and workspace.k == k and m <= workspace.max_m, "workspace does not fit this call")
    out, ldy = _output(out, m, n, dev)
    nat = workspace.sf_natural
    with torch.cuda.device(dev):
        _sm100._check(_lib().adg_o2_linear(
            a_int8.data_ptr(), a_scale.data_ptr(), w_mxfp4.data_ptr(), w_sf_tiled.data_ptr(), workspace.operand.data_ptr(),
            workspace.sf_tiled.data_ptr(), nat.data_ptr() if nat is not None else None,
            workspace.counters.data_ptr() if workspace.counters is not None else None, out.data_ptr(), m, n, k, ldy, _stream(out)))
    return out


class O1xWeights:
    """W prepared for the exact-integer O1 variant: the row-shifted INT8 image, one factor per W row, the
    list of column blocks that must take the literal path, and the literal path's own INT8 image."""

    def __init__(self, w_mxfp4, w_scale):
        import torch

        n, kh = w_mxfp4.shape
        k = kh * 2
        dev = w_mxfp4.device
        _operand(w_mxfp4, "W_mxfp4", torch.uint8)
        _operand(w_scale, "W_scale", torch.uint8, (n, k // 32), dev)
        self.n, self.k = n, k
        self.w_scale = w_scale
        self.w_int8 = mxfp4_to_int8(w_mxfp4)
        self.w_int8x = torch.empty((n, k), dtype=torch.int8, device=dev)
        self.col_factor = torch.empty((n,), dtype=torch.float32, device=dev)
        self.workspace = torch.zeros(((int(_lib().adg_o1x_workspace_bytes(n)) + 15) // 16 * 4,), dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            _sm100._check(_lib().adg_o1x_prepare_weight(
                w_mxfp4.data_ptr(), w_scale.data_ptr(), self.w_int8x.data_ptr(), self.col_factor.data_ptr(),
                self.workspace.data_ptr(), n, k, _stream(w_mxfp4)))

    def ineligible_rows(self) -> int:
        """Number of W rows (output columns) whose scale-code spread exceeds 3 (synchronises)."""
        import torch

        rows = ctypes.c_int64(0)
        with torch.cuda.device(self.w_int8.device):
            _sm100._check(_lib().adg_o1x_ineligible_rows(self.workspace.data_ptr(), _stream(self.w_int8), ctypes.byref(rows)))
        return int(rows.value)


def gemm_o1x(a_int8, a_scale, weights: O1xWeights, out=None):
    """The exact-integer O1 variant (``adg_gemm_o1x``): NOT the O1 recurrence; see the header."""
    import torch

    m, k = a_int8.shape
    dev = a_int8.device
    _operand(a_int8, "A_int8", torch.int8)
    _operand(a_scale, "A_scale", torch.float32, (m,), dev)
    _require(k == weights.k and weights.w_int8.device == dev, "weights do not match A")
    out, ldy = _output(out, m, weights.n, dev)
    with torch.cuda.device(dev):
        _sm100._check(_lib().adg_gemm_o1x(
            a_int8.data_ptr(), a_scale.data_ptr(), weights.w_int8x.data_ptr(), weights.col_factor.data_ptr(),
            weights.workspace.data_ptr(), weights.w_int8.data_ptr(), weights.w_scale.data_ptr(), out.data_ptr(),
            m, weights.n, k, ldy, _stream(out)))
    return out


def check_status(device=None):
    """Synchronise torch's current stream and raise if a kernel reported a bounded-wait timeout."""
    import torch

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _sm100._check(_lib().adg_check_status(torch.cuda.current_stream(dev).cuda_stream))


class HostSession:
    """Weights resident on the device, activations and results in host memory
    (``adg_session_*`` of the C ABI).  numpy arrays or CPU torch tensors are accepted."""

    def __init__(self, variant: str, max_m: int, w_mxfp4, w_scale):
        self._handle = ctypes.c_void_p()
        self.variant = variant
        self.n, kh = w_mxfp4.shape
        self.k = kh * 2
        self.max_m = max_m
        _sm100._check(_lib().adg_session_create(
            ctypes.byref(self._handle), _sm100._VARIANTS[variant], max_m, self.n, self.k,
            _host_ptr(w_mxfp4), _host_ptr(w_scale)))

    def run(self, a_int8, a_scale, y_out):
        m = a_int8.shape[0]
        _sm100._check(_lib().adg_session_run(self._handle, _host_ptr(a_int8), _host_ptr(a_scale), m, _host_ptr(y_out)))
        return y_out

    def submit(self, a_int8, a_scale, y_out):
        """Enqueue one pass and return at once; the host buffers must be pinned and stay untouched
        until :meth:`wait`.  Passes of different sessions overlap (each session has its own stream)."""
        m = a_int8.shape[0]
        _sm100._check(_lib().adg_session_submit(self._handle, _host_ptr(a_int8), _host_ptr(a_scale), m, _host_ptr(y_out)))
        return y_out

    def wait(self):
        _sm100._check(_lib().adg_session_wait(self._handle))

    def close(self):
        if self._handle:
            _lib().adg_session_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _host_ptr(x):
    if hasattr(x, "data_ptr"):
        _require(not x.is_cuda and x.is_contiguous(), "expected a contiguous host tensor")
        return x.data_ptr()
    _require(x.flags["C_CONTIGUOUS"], "expected a C-contiguous array")
    return x.ctypes.data
