"""CPU oracle for the O0/O1/O2 quantized-GEMM path (numpy restatement).

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is judged against.  It is
imported by the test-suite, by the smoke check and by the CPU-baseline leg of the benchmark; the
shipped package never imports it and has no CPU fallback.

Every function restates one piece of the reference project's Python semantic reference and cites
the file:line it follows (paths are relative to the reference project's root).  The restatement is
pinned against golden vectors produced by importing that reference (``tests/golden/make_golden.py``)
and against the scalar known-answer tables of ``tests/unit/test_mxfp4_codec.py``.

One deliberate difference, found while pinning: the reference's *tensor* quantizer takes the block
exponent as ``floor(log2(amax))`` evaluated in FP32 (``python/adangel/quantization/mxfp4.py:162``),
which rounds up by one for an ``amax`` a few ulps below a power of two, whereas the reference's own
scalar helper (``mxfp4.py:73``, ``math.frexp``) and its CUDA kernel (``csrc/sm120/o2_cutlass.cu:237``,
``ilogbf``) are exact.  ``block_exponent`` here is exact; ``block_exponent_log2_fp32`` reproduces
the FP32-log2 variant so tests can classify any block where the two disagree.
"""

from __future__ import annotations

import numpy as np

GROUP_SIZE = 32  # python/adangel/quantization/mxfp4.py:15
UE8M0_BIAS = 127  # mxfp4.py:16
UE8M0_NAN = 255  # mxfp4.py:17

# mxfp4.py:12-14
E2M1_POSITIVE = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_DECODE = np.concatenate([E2M1_POSITIVE, -E2M1_POSITIVE]).astype(np.float32)
E2M1_TO_INT8_BASE = np.array(
    [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], dtype=np.int8
)


# --------------------------------------------------------------------------------------------
# INT8 per-row activation codec  (python/adangel/quantization/int8.py)
# --------------------------------------------------------------------------------------------

def quantize_int8_per_row(x: np.ndarray):
    """int8.py:6-17 — scale = row amax / 127 (1 for an all-zero row), round-half-even, clamp ±127."""
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    if x32.ndim != 2:
        raise ValueError("activation must be rank-2")
    if not np.isfinite(x32).all():
        raise ValueError("activation contains NaN/Inf")
    amax = np.abs(x32).max(axis=1)
    scale = np.where(amax == 0, np.float32(1.0), amax / np.float32(127.0)).astype(np.float32)
    q = np.rint(x32 / scale[:, None]).clip(-127, 127).astype(np.int8)
    return q, scale


def dequantize_int8_per_row(q: np.ndarray, scale: np.ndarray, dtype=np.float32):
    """int8.py:20-28 — one FP32 multiply, then (optionally) round-to-nearest into ``dtype``."""
    if q.dtype != np.int8 or q.ndim != 2:
        raise ValueError("quantized activation must be rank-2 int8")
    if scale.dtype != np.float32 or scale.shape != (q.shape[0],):
        raise ValueError("activation scale must be row-shaped fp32")
    with np.errstate(over="ignore"):
        return (q.astype(np.float32) * scale[:, None]).astype(dtype)


# --------------------------------------------------------------------------------------------
# MXFP4 (E2M1 + UE8M0, K32) codec  (python/adangel/quantization/mxfp4.py)
# --------------------------------------------------------------------------------------------

def block_exponent(amax: np.ndarray) -> np.ndarray:
    """Exact ``floor(log2(amax)) - 2`` clamped to ±127, 0 for an all-zero block.

    Follows the scalar helper ``choose_ue8m0_scale_code`` (mxfp4.py:62-74, ``math.frexp``) and the
    reference CUDA kernel (``csrc/sm120/o2_cutlass.cu:235-239``, ``ilogbf``).
    """
    amax = np.asarray(amax, dtype=np.float32)
    _, e = np.frexp(np.where(amax == 0, np.float32(1.0), amax))
    exps = (e.astype(np.int32) - 1) - 2
    exps = np.where(amax == 0, 0, exps)
    return np.clip(exps, -127, 127).astype(np.int32)


def block_exponent_log2_fp32(amax: np.ndarray) -> np.ndarray:
    """The FP32 ``floor(log2(.))`` variant of mxfp4.py:162-163 (differs just below powers of two)."""
    amax = np.asarray(amax, dtype=np.float32)
    safe = np.where(amax == 0, np.float32(1.0), amax)
    exps = np.floor(np.log2(safe, dtype=np.float32)) - 2
    exps = np.where(amax == 0, 0, exps)
    return np.clip(exps, -127, 127).astype(np.int32)


def encode_e2m1(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even onto the E2M1 grid with saturation; returns 4-bit codes.

    Equivalent to the nearest-level / even-tie-break selection of mxfp4.py:168-177 and to the
    threshold form of ``include/adangel/data_types.cuh:26-39``.  The sign bit is set for every
    negative value, including one that rounds to zero; ``-0.0`` encodes as 0 (``normalized < 0``).
    """
    v = np.asarray(values, dtype=np.float32)
    mag = np.abs(v)
    code = (
        (mag > 0.25).astype(np.uint8)
        + (mag >= 0.75)
        + (mag > 1.25)
        + (mag >= 1.75)
        + (mag > 2.5)
        + (mag >= 3.5)
        + (mag > 5.0)
    ).astype(np.uint8)
    return code | ((v < 0).astype(np.uint8) << 3)


def pack_e2m1(codes: np.ndarray) -> np.ndarray:
    """mxfp4.py:98-109,179 — even K in the low nibble, odd K in the high nibble."""
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """mxfp4.py:183-190."""
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def quantize_mxfp4(x: np.ndarray, row_chunk: int = 1024, exponent=block_exponent):
    """mxfp4.py:147-180 — per (row, K32 block): UE8M0 scale code and packed E2M1 codes.

    Rows are independent, so the work is done in row chunks to bound memory.
    """
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    if x32.ndim != 2 or x32.shape[1] % GROUP_SIZE:
        raise ValueError("x must be rank-2 and K must be divisible by 32")
    rows, cols = x32.shape
    packed = np.empty((rows, cols // 2), dtype=np.uint8)
    scale_codes = np.empty((rows, cols // GROUP_SIZE), dtype=np.uint8)
    for r0 in range(0, rows, row_chunk):
        blocks = x32[r0:r0 + row_chunk].reshape(-1, cols // GROUP_SIZE, GROUP_SIZE)
        amax = np.abs(blocks).max(axis=-1)
        if not np.isfinite(amax).all():
            raise ValueError("MXFP4 input contains NaN/Inf")
        exps = exponent(amax)
        scale_codes[r0:r0 + row_chunk] = (exps + UE8M0_BIAS).astype(np.uint8)
        scales = np.ldexp(np.float32(1.0), exps).astype(np.float32)[..., None]
        with np.errstate(over="ignore"):
            normalized = blocks / scales
        codes = encode_e2m1(normalized).reshape(blocks.shape[0], cols)
        packed[r0:r0 + row_chunk] = pack_e2m1(codes)
    return packed, scale_codes


def decode_ue8m0(scale_codes: np.ndarray) -> np.ndarray:
    """mxfp4.py:193-199 — 2**(code-127) in FP32; code 255 (NaN) is forbidden."""
    scale_codes = np.asarray(scale_codes)
    if scale_codes.dtype != np.uint8:
        raise ValueError("UE8M0 scales must be uint8")
    if (scale_codes == UE8M0_NAN).any():
        raise ValueError("UE8M0 NaN scale code 255 is forbidden")
    return np.ldexp(np.float32(1.0), scale_codes.astype(np.int32) - UE8M0_BIAS).astype(np.float32)


def decode_e2m1(codes: np.ndarray) -> np.ndarray:
    """mxfp4.py:202-205."""
    return E2M1_DECODE[np.asarray(codes, dtype=np.int64)]


def mxfp4_to_int8_base(packed: np.ndarray) -> np.ndarray:
    """mxfp4.py:208-212 — exact ``2*E2M1`` INT8 image of every nibble (the O1 weight conversion)."""
    return E2M1_TO_INT8_BASE[unpack_e2m1(packed).astype(np.int64)]


def dequantize_mxfp4(packed: np.ndarray, scale_codes: np.ndarray, dtype=np.float32):
    """mxfp4.py:215-224 — FP32 ``e2m1 * 2**(s-127)`` then round-to-nearest into ``dtype``."""
    values = decode_e2m1(unpack_e2m1(packed))
    rows, cols = values.shape
    if cols % GROUP_SIZE:
        raise ValueError("unpacked K must be divisible by 32")
    if scale_codes.shape != (rows, cols // GROUP_SIZE):
        raise ValueError("scale shape does not match packed values")
    scaled = values.reshape(rows, -1, GROUP_SIZE) * decode_ue8m0(scale_codes)[..., None]
    with np.errstate(over="ignore"):
        return scaled.reshape(rows, cols).astype(dtype)


# --------------------------------------------------------------------------------------------
# The three variants  (python/adangel/reference/o0.py, o1.py, o2.py)
# --------------------------------------------------------------------------------------------

def run_o0(a_int8, a_scale, w_mxfp4, w_scale):
    """reference/o0.py:9-24 — both operands rounded to FP16, FP32 product/accumulate."""
    a16 = dequantize_int8_per_row(a_int8, a_scale, np.float16)
    w16 = dequantize_mxfp4(w_mxfp4, w_scale, np.float16)
    y = a16.astype(np.float32) @ w16.astype(np.float32).T
    return {"output": y, "converted_weight": w16, "converted_activation": a16}


def o1_partials(a_int8, w_int8):
    """The exact INT32 K32 partial sums ``P[m, n, g]`` of reference/o1.py:17-18."""
    m, k = a_int8.shape
    n = w_int8.shape[0]
    groups = k // GROUP_SIZE
    a = a_int8.astype(np.int32).reshape(m, groups, GROUP_SIZE)
    w = w_int8.astype(np.int32).reshape(n, groups, GROUP_SIZE)
    return np.einsum("mgk,ngk->mng", a, w, dtype=np.int32)


def run_o1(a_int8, a_scale, w_mxfp4, w_scale):
    """reference/o1.py:8-29 — per K32 group: INT32 dot, FP32 scale ``(A_scale*2**(s-127))*0.5``,
    FP32 multiply and FP32 add into the output, groups in ascending order.

    The INT32 dot is evaluated as an FP32 matmul of integer-valued operands: every product is at
    most 127*12 and every partial sum at most 32*127*12 = 48768 < 2**24, so each intermediate is an
    exactly representable integer in any summation order and the result equals the INT32 dot
    (the same argument as ``scripts/validate_o1.py:25-46``).
    """
    w_int8 = mxfp4_to_int8_base(w_mxfp4)
    m, k = a_int8.shape
    n = w_int8.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    w_scales = decode_ue8m0(w_scale)
    a_f = a_int8.astype(np.float32)
    w_f = w_int8.astype(np.float32)
    half = np.float32(0.5)
    for g in range(k // GROUP_SIZE):
        sl = slice(g * GROUP_SIZE, (g + 1) * GROUP_SIZE)
        partial = a_f[:, sl] @ w_f[:, sl].T
        scale = (a_scale[:, None] * w_scales[:, g][None, :]) * half
        y += partial * scale
    return {"output": y, "converted_weight": w_int8, "converted_activation": None}


def run_o2(a_int8, a_scale, w_mxfp4, w_scale, exponent=block_exponent):
    """reference/o2.py:9-25 — A dequantized to FP32, re-quantized to MXFP4, both sides dequantized
    to FP32 and multiplied with FP32 accumulation."""
    activation = dequantize_int8_per_row(a_int8, a_scale, np.float32)
    a_mx, a_sc = quantize_mxfp4(activation, exponent=exponent)
    a_deq = dequantize_mxfp4(a_mx, a_sc, np.float32)
    w_deq = dequantize_mxfp4(w_mxfp4, w_scale, np.float32)
    y = a_deq @ w_deq.T
    return {"output": y, "converted_weight": None, "converted_activation": (a_mx, a_sc)}


def prepare_weights(w_mxfp4, w_scale):
    """The weight-side work of the three variants, done once (the steady-state case): FP16-rounded
    W for O0, the INT8 image and FP32 group scales for O1, FP32 dequantized W for O2."""
    w_int8 = mxfp4_to_int8_base(w_mxfp4)
    return {
        "w16": dequantize_mxfp4(w_mxfp4, w_scale, np.float16).astype(np.float32),
        "w_int8_f32": w_int8.astype(np.float32),
        "w_scales": decode_ue8m0(w_scale),
        "w_deq": dequantize_mxfp4(w_mxfp4, w_scale, np.float32),
    }


def steady_state_step(a_int8, a_scale, prepared):
    """One steady-state pass of O0, O1 and O2 on prepared weights: per variant the activation-side
    conversion plus the GEMM, exactly the arithmetic of run_o0 / run_o1 / run_o2."""
    a16 = dequantize_int8_per_row(a_int8, a_scale, np.float16)
    y0 = a16.astype(np.float32) @ prepared["w16"].T
    m, k = a_int8.shape
    y1 = np.zeros((m, prepared["w16"].shape[0]), dtype=np.float32)
    a_f = a_int8.astype(np.float32)
    half = np.float32(0.5)
    for g in range(k // GROUP_SIZE):
        sl = slice(g * GROUP_SIZE, (g + 1) * GROUP_SIZE)
        partial = a_f[:, sl] @ prepared["w_int8_f32"][:, sl].T
        y1 += partial * ((a_scale[:, None] * prepared["w_scales"][:, g][None, :]) * half)
    act = dequantize_int8_per_row(a_int8, a_scale, np.float32)
    a_mx, a_sc = quantize_mxfp4(act)
    y2 = dequantize_mxfp4(a_mx, a_sc, np.float32) @ prepared["w_deq"].T
    return y0, y1, y2


def mse_fp64(output, reference) -> float:
    """python/adangel/benchmark/metrics.py:42-50."""
    if output.shape != reference.shape:
        raise ValueError("MSE operands have different shapes")
    if not np.isfinite(output).all() or not np.isfinite(reference).all():
        raise ValueError("NaN/Inf found in experiment output")
    d = output.astype(np.float64) - reference.astype(np.float64)
    return float(np.mean(d * d))


# --------------------------------------------------------------------------------------------
# Scale-factor physical layout consumed by the block-scaled MMA
# --------------------------------------------------------------------------------------------

def tiled_scale_shape(rows: int, k: int):
    """Padded extent of the tiled layout: rows to a multiple of 256, K32 blocks to a multiple of 8."""
    groups = k // GROUP_SIZE
    return ((rows + 255) // 256) * 256, ((groups + 7) // 8) * 8


def tile_scale_factors(natural: np.ndarray) -> np.ndarray:
    """Natural ``[rows, K/32]`` scale bytes -> the 512-byte-atom layout the tensor core reads.

    One atom covers 128 rows x 4 K32 blocks; inside it byte ``(r % 32) * 16 + (r // 32) * 4 + kb``
    holds row ``r`` / block ``kb``; atoms are ordered row-block major, K-atom minor.  This is the
    permutation the reference performs in ``adangel_o2_repack_scale``
    (``csrc/sm120/o2_cutlass.cu:261-274``) for its scale-factor atom; padding bytes are zero.
    """
    rows, groups = natural.shape
    prow, pgroups = tiled_scale_shape(rows, groups * GROUP_SIZE)
    padded = np.zeros((prow, pgroups), dtype=np.uint8)
    padded[:rows, :groups] = natural
    t = padded.reshape(prow // 128, 4, 32, pgroups // 4, 4)  # [rb, j, r, ka, kb]
    t = t.transpose(0, 3, 2, 1, 4)  # [rb, ka, r, j, kb]
    return np.ascontiguousarray(t).reshape(-1)


# --------------------------------------------------------------------------------------------
# Synthetic stand-in for the reference's prepared traces
# --------------------------------------------------------------------------------------------

def canonical_inputs(m: int, n: int, k: int, seed: int = 20250805):
    """Seeded synthetic inputs with the canonical distributions: A ~ N(0,1) with 0.5 % of the K
    channels scaled x20, W ~ N(0, 0.02); A quantized per row to INT8, W to MXFP4.

    The float draws use torch's CPU generator (``randn``, ``randperm``, ``randn`` in this order) so
    that every consumer of the same seed sees the same bits.
    """
    import torch

    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    idx = torch.randperm(k, generator=g)[: max(1, round(0.005 * k))]
    a[:, idx] *= 20.0
    w = torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02
    a_int8, a_scale = quantize_int8_per_row(a.numpy())
    w_mxfp4, w_scale = quantize_mxfp4(w.numpy())
    return a_int8, a_scale, w_mxfp4, w_scale


# --------------------------------------------------------------------------------------------
# o1x: the exact-integer variant of O1 (an addition of the B200 build; the reference has no such
# variant -- its O1 is run_o1 above, python/adangel/reference/o1.py:8-29)
# --------------------------------------------------------------------------------------------

O1X_MAX_SPREAD = 3
O1X_BLOCK = 128  # output columns are handed to the literal recurrence in blocks of this many


def o1x_prepare(w_mxfp4, w_scale):
    """Per W row: the smallest scale code over the blocks that hold a non-zero nibble, whether the row's
    code spread allows one exponent (<= 3, so that 12 * 2**3 = 96 still fits INT8), and the INT8 image
    ``2*e2m1 << (code - min code)`` (zero for an ineligible row)."""
    n, kh = w_mxfp4.shape
    groups = kh * 2 // GROUP_SIZE
    base = mxfp4_to_int8_base(w_mxfp4).astype(np.int32).reshape(n, groups, GROUP_SIZE)
    nonzero = (base != 0).any(axis=2)
    codes = w_scale.astype(np.int32)
    emin = np.where(nonzero, codes, 255).min(axis=1)
    emax = np.where(nonzero, codes, 0).max(axis=1)
    empty = emax < emin
    emin = np.where(empty, 127, emin)
    eligible = empty | (emax - emin <= O1X_MAX_SPREAD)
    shift = np.clip(codes - emin[:, None], 0, O1X_MAX_SPREAD)
    shifted = np.where(eligible[:, None, None], base << shift[:, :, None], 0).reshape(n, kh * 2)
    factor = np.where(eligible, np.ldexp(np.float64(1.0), emin - 128), 0.0).astype(np.float32)
    return shifted.astype(np.int8), factor, eligible


def run_o1x(a_int8, a_scale, w_mxfp4, w_scale):
    """``y = RN(float32_rn(S) * RN(A_scale[m] * 2**(emin[n]-128)))`` with ``S`` the exact integer sum over
    all of K; 128-column blocks that contain an ineligible W row take run_o1's recurrence instead."""
    w_shift, factor, eligible = o1x_prepare(w_mxfp4, w_scale)
    sums = a_int8.astype(np.int64) @ w_shift.astype(np.int64).T  # exact
    assert np.abs(sums).max(initial=0) < 2**31
    scale = a_scale.astype(np.float32)[:, None] * factor[None, :]
    y = sums.astype(np.float32) * scale
    n = w_mxfp4.shape[0]
    bad_blocks = sorted({int(i) // O1X_BLOCK for i in np.nonzero(~eligible)[0]})
    if bad_blocks:
        literal = run_o1(a_int8, a_scale, w_mxfp4, w_scale)["output"]
        for b in bad_blocks:
            y[:, b * O1X_BLOCK:min(n, (b + 1) * O1X_BLOCK)] = literal[:, b * O1X_BLOCK:min(n, (b + 1) * O1X_BLOCK)]
    return {"output": y, "converted_weight": w_shift, "column_factor": factor, "ineligible_rows": int((~eligible).sum())}
