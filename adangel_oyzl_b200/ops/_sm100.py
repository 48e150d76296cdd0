"""ctypes binding of ``libadangel_b200.so`` with the function surface of the reference's native
extension module (``csrc/bindings.cpp:84-103``): ``capabilities``, ``run_o0/run_o1/run_o2``,
``benchmark`` and ``verify_layout``, taking and returning torch CUDA tensors.

PyTorch is used for device memory and the current stream only; all computation happens in the
library's CUDA kernels.  Errors reported by the library surface as ``RuntimeError``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parents[1] / "lib" / "libadangel_b200.so"
_lib = None

DEFAULT_CONVERSION_INNER_REPEATS = 100  # include/adangel/kernel_api.h:9 of the reference
_MODES = {"conversion_only": 0, "compute_only": 1, "cold": 2, "steady_state": 3}
_VARIANTS = {"o0": 0, "o1": 1, "o2": 2, "o1x": 3}  # o1x: the exact-integer O1 variant, only ever by name
BENCH_FUSE_ACTIVATION = 1
BENCH_O1_SPLIT_ACTIVATION = 2
BENCH_FLUSH_L2 = 4
L2_FLUSH_BYTES = 256 << 20  # more than the 126 MB L2 of a B200
PLAN_O1_BF16, PLAN_FUSED_ACTIVATION, PLAN_PARTIAL_DUMP = 1, 2, 4
_STAGE_BITS = (("weight_conversion", 1), ("activation_conversion", 2), ("gemm", 4), ("total", 8))


class BenchArgs(ctypes.Structure):
    """``adg_bench_args`` of include/adangel_b200.h."""

    _fields_ = [
        ("variant", c_int32), ("mode", c_int32),
        ("M", c_int32), ("N", c_int32), ("K", c_int32),
        ("warmup", c_int32), ("repeats", c_int32), ("conversion_inner_repeats", c_int32),
        ("a_int8", c_void_p), ("a_scale", c_void_p), ("w_mxfp4", c_void_p), ("w_scale", c_void_p),
        ("output", c_void_p), ("conv_weight", c_void_p), ("conv_act", c_void_p),
        ("conv_act_sf", c_void_p), ("conv_act_sf_tiled", c_void_p),
        ("t_weight", POINTER(c_float)), ("t_activation", POINTER(c_float)),
        ("t_gemm", POINTER(c_float)), ("t_total", POINTER(c_float)),
        ("stages_out", c_uint32), ("stream", c_void_p),
        ("conv_weight_bf16", c_void_p), ("conv_act_bf16", c_void_p), ("range_flag", c_void_p),
        ("flags", c_uint32), ("row_counters", c_void_p),
        ("o1x_col_factor", c_void_p), ("o1x_workspace", c_void_p), ("o1x_w_int8", c_void_p),
        ("l2_flush", c_void_p), ("l2_flush_bytes", c_int64),
    ]


class PlanDesc(ctypes.Structure):
    """``adg_plan_desc`` of include/adangel_b200.h."""

    _fields_ = [
        ("tile_m", c_int32), ("tile_n", c_int32), ("stages", c_int32), ("accumulator_stages", c_int32),
        ("threads", c_int32), ("cluster", c_int32), ("mma_m", c_int32), ("mma_n", c_int32), ("mma_k", c_int32),
        ("persistent", c_int32), ("fused_activation", c_int32),
        ("kernel_symbol", ctypes.c_char * 64), ("mma_family", ctypes.c_char * 96),
    ]


MAX_PEER_BLOCKS = 16
PEER_HANDLE_BYTES = 64


class PeerBlocks(ctypes.Structure):
    """``adg_peer_blocks`` of include/adangel_b200.h."""

    _fields_ = [("src", c_void_p * MAX_PEER_BLOCKS), ("col0", c_int * MAX_PEER_BLOCKS), ("width", c_int * MAX_PEER_BLOCKS),
                ("count", c_int)]


_SIGNATURES = {
    "adg_abi_version": (c_int, []),
    "adg_last_error": (c_char_p, []),
    "adg_capabilities": (c_uint32, []),
    "adg_device_info": (c_int, [c_char_p, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "adg_check_status": (c_int, [c_void_p]),
    "adg_plan_info": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(PlanDesc)]),
    "adg_fused_workspace_bytes": (c_int64, [c_int64]),
    "adg_o0_linear": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_void_p]),
    "adg_o2_linear": (c_int, [c_void_p] * 9 + [c_int, c_int, c_int, c_int, c_void_p]),
    "adg_o1x_workspace_bytes": (c_int64, [c_int64]),
    "adg_o1x_prepare_weight": (c_int, [c_void_p] * 5 + [c_int64, c_int64, c_void_p]),
    "adg_o1x_ineligible_rows": (c_int, [c_void_p, c_void_p, POINTER(c_int64)]),
    "adg_gemm_o1x": (c_int, [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_void_p]),
    "adg_o2_linear_noalloc_status": (c_int, [c_void_p]),
    "adg_o2_linear_noalloc_status_words": (c_int, [POINTER(c_void_p), POINTER(c_int)]),
    "adg_mxfp4_to_fp16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_int8_to_fp16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_mxfp4_to_int8": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_mxfp4_to_bf16_scaled": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_int8_to_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_o2_tiled_scale_bytes": (c_int64, [c_int64, c_int64]),
    "adg_o2_quantize_activation": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_o2_tile_scales": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_quantize_int8_per_row": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_quantize_mxfp4": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "adg_gemm_o0": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "adg_gemm_o1": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "adg_gemm_o1_packed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "adg_gemm_o1_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "adg_o1_linear": (c_int, [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_void_p]),
    "adg_gemm_o2": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "adg_o2_linear_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int]),
    "adg_benchmark": (c_int, [POINTER(BenchArgs)]),
    "adg_verify_layout": (c_int, [POINTER(c_int), POINTER(c_float)]),
    "adg_peer_export": (c_int, [c_void_p, c_void_p, POINTER(c_uint64)]),
    "adg_peer_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "adg_peer_close": (c_int, [c_void_p]),
    "adg_gather_columns_pull": (c_int, [POINTER(PeerBlocks), c_void_p, c_int, c_int64, c_void_p]),
    "adg_session_create": (c_int, [POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "adg_session_run": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "adg_session_submit": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "adg_session_wait": (c_int, [c_void_p]),
    "adg_session_destroy": (None, [c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def library():
    """dlopen the native library (once) and attach argument/return types."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise OSError(f"{_LIB_PATH} is not built; run `python -m adangel_oyzl_b200.build`")
        lib = ctypes.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(library().adg_last_error().decode("utf-8", "replace"))


def capabilities() -> dict:
    bits = library().adg_capabilities()
    return {
        "compiled_sm100a": bool(bits & 0x01),
        "o0_fp16_tc": bool(bits & 0x02),
        "o1_int8_tc": bool(bits & 0x04),
        "o2_mxf4_block_scale": bool(bits & 0x08),
        "o2_cutlass_tiled": bool(bits & 0x10),  # key kept for schema compatibility: the tiled production O2 kernel
        "status": "O0/O1/O2 production kernels are implemented (hand-written sm_100a)",
    }


# ---- input contract (reference csrc/common/validation.cu:5-33) -------------------------------------

def validate_cuda_inputs(a_int8, a_scale, w_mxfp4, w_scale):
    import torch

    tensors = (a_int8, a_scale, w_mxfp4, w_scale)
    if not all(t.is_cuda for t in tensors):
        raise RuntimeError("all inputs must be CUDA tensors")
    if a_int8.dim() != 2:
        raise RuntimeError("A_int8 must be rank-2")
    if a_scale.dim() != 1:
        raise RuntimeError("A_scale must be rank-1")
    if w_mxfp4.dim() != 2:
        raise RuntimeError("W_mxfp4 must be rank-2")
    if w_scale.dim() != 2:
        raise RuntimeError("W_scale must be rank-2")
    if len({t.device for t in tensors}) != 1:
        raise RuntimeError("all inputs must be on the same CUDA device")
    if a_int8.dtype != torch.int8:
        raise RuntimeError("A_int8 must be int8")
    if a_scale.dtype != torch.float32:
        raise RuntimeError("A_scale must be fp32")
    if w_mxfp4.dtype != torch.uint8:
        raise RuntimeError("W_mxfp4 must be uint8")
    if w_scale.dtype != torch.uint8:
        raise RuntimeError("W_scale must be uint8")
    if not all(t.is_contiguous() for t in tensors):
        raise RuntimeError("all inputs must be contiguous")
    m, k = a_int8.shape
    n = w_mxfp4.shape[0]
    if m <= 0 or n <= 0 or k <= 0:
        raise RuntimeError("M, N, and K must be positive")
    if k % 64:
        raise RuntimeError("K must be divisible by 64")
    if tuple(a_scale.shape) != (m,):
        raise RuntimeError("invalid A_scale shape")
    if tuple(w_mxfp4.shape) != (n, k // 2):
        raise RuntimeError("invalid W_mxfp4 shape")
    if tuple(w_scale.shape) != (n, k // 32):
        raise RuntimeError("invalid W_scale shape")
    return int(m), int(n), int(k)


def _timing_metadata(mode: str, inner: int) -> dict:
    # the strings the runner validates (reference csrc/sm120/o0_gemm.cu:330-345)
    return {
        "strategy": "conversion_amortized_end_to_end_direct",
        "conversion_stage_timing": "isolated_batched_cuda_event_average",
        "conversion_inner_repeats": inner,
        "conversion_only_total_timing": "batched_cuda_event_average",
        "end_to_end_total_timing": "direct_single_path",
        "mode_total_timing": "batched_cuda_event_average" if mode == "conversion_only" else "direct_single_path",
        "mode_total_inner_repeats": inner if mode == "conversion_only" else 1,
        "component_and_total_measured_separately": True,
    }


def plan_info(variant: str, m: int, n: int, k: int, o1_bf16: bool = False, fused: bool = False,
              partial_dump: bool = False) -> dict:
    """The planner's choice for a shape, asked of the library (``adg_plan_info``); needs a device."""
    desc = PlanDesc()
    flags = (PLAN_O1_BF16 if o1_bf16 else 0) | (PLAN_FUSED_ACTIVATION if fused else 0) | (PLAN_PARTIAL_DUMP if partial_dump else 0)
    _check(library().adg_plan_info(_VARIANTS[variant], flags, m, n, k, ctypes.byref(desc)))
    return {
        "kernel_symbol": desc.kernel_symbol.decode(),
        "mma_family": desc.mma_family.decode(),
        "tile": [desc.tile_m, desc.tile_n],
        "stages": desc.stages,
        "accumulator_stages": desc.accumulator_stages,
        "threads": desc.threads,
        "cluster": [desc.cluster, 1, 1],
        "mma_shape": [desc.mma_m, desc.mma_n, desc.mma_k],
        "persistent": bool(desc.persistent),
        "fused_activation_conversion": bool(desc.fused_activation),
    }


def kernel_metadata(variant: str, m: int, n: int, k: int, o1_bf16: bool = False, fused: bool = False) -> dict:
    """The ``kernel`` dictionary of a result (the reference builds its own by hand per variant,
    csrc/sm120/o0_gemm.cu:300-328): constant facts plus the planner's choice from :func:`plan_info`."""
    meta = {
        "library": "hand-written sm_100a (no CUTLASS, no cuBLAS)",
        "tensor_core": True,
        "data_movement": "TMA",
        "accumulator": "tensor memory (tcgen05)",
        "global_partial_buffer": False,
        "output_stores_per_element": 1,
        "group_size": 32,
    }
    meta.update(plan_info(variant, m, n, k, o1_bf16=o1_bf16, fused=fused))
    if variant == "o1":
        meta["partial_rescale"] = "per-K32, FP32 registers"
        meta["accumulator"] = ("FP32 partial in tensor memory, FP32 accumulate in registers" if o1_bf16 and m > 64
                               else "INT32 partial in tensor memory, FP32 accumulate in registers")
    elif variant == "o1x":
        meta["partial_rescale"] = "none: INT32 accumulation over all of K, one scaling per output element"
        meta["accumulator"] = "INT32 in tensor memory"
    elif variant == "o2":
        meta["scale_format"] = "UE8M0"
        meta["weight_copy"] = False
    return meta


def benchmark(variant, mode, a_int8, a_scale, w_mxfp4, w_scale, warmup, repeats,
              conversion_inner_repeats=DEFAULT_CONVERSION_INNER_REPEATS, *, fuse_activation=False,
              o1_split_activation_stage=False, flush_l2=False):
    """One variant/mode under the reference's timing protocol (``adangel_benchmark_o{0,1,2}``).

    The positional signature is the reference's.  Keyword-only additions: ``fuse_activation`` (O0/O2, cold and
    steady-state modes, M > 64: the activation conversion runs inside the GEMM kernel, so the ``gemm`` stage is
    that one kernel and ``activation_conversion`` is reported from its isolated batches only; off by default:
    the two-kernel sequence is faster at every measured shape);
    ``o1_split_activation_stage`` (O1 on BF16 operands: report the INT8 -> BF16 conversion as an
    ``activation_conversion`` stage instead of inside ``gemm``; off by default because the reference's O1 has
    no such stage); ``flush_l2`` (overwrite a 256 MiB buffer before every directly timed iteration, outside its
    events, so that operands come from HBM: how the weight-streaming decode shapes are measured against the HBM
    roofline -- the reference's protocol leaves the L2 warm).  ``variant="o1x"`` runs the exact-integer O1 variant; its result carries
    ``o1x_ineligible_rows``."""
    import torch

    lib = library()
    if variant not in _VARIANTS:
        raise RuntimeError(
            f"The {variant} SM100 production benchmark is not implemented; reference code must not be "
            "used for formal timing.")
    if mode not in _MODES:
        raise RuntimeError(f"unknown timing mode: {mode}")
    if warmup < 0:
        raise RuntimeError("warmup must be non-negative")
    if repeats <= 0:
        raise RuntimeError("repeats must be positive")
    if conversion_inner_repeats <= 1:
        raise RuntimeError("conversion_inner_repeats must exceed one")
    m, n, k = validate_cuda_inputs(a_int8, a_scale, w_mxfp4, w_scale)
    device = a_int8.device
    if variant == "o2":
        # reference csrc/sm120/o2_cutlass.cu:383-386 (outside the timed region)
        if not bool(torch.isfinite(a_scale).all()):
            raise RuntimeError("A_scale contains NaN/Inf")
        if bool(torch.any(w_scale == 255)):
            raise RuntimeError("W_scale contains forbidden UE8M0 NaN code 255")

    def empty(shape, dtype):
        return torch.empty(shape, dtype=dtype, device=device)

    output = empty((m, n), torch.float32)
    conv_weight = conv_act = conv_act_sf = conv_act_sf_tiled = None
    conv_weight_bf16 = conv_act_bf16 = range_flag = None
    row_counters = o1x_col_factor = o1x_workspace = o1x_w_int8 = None
    fused = bool(fuse_activation) and variant in ("o0", "o2") and m > 64 and mode in ("cold", "steady_state")
    if fused:
        row_counters = torch.zeros((lib.adg_fused_workspace_bytes(m) // 4,), dtype=torch.int32, device=device)
    if variant == "o1x":
        conv_weight = empty((n, k), torch.int8)
        o1x_w_int8 = empty((n, k), torch.int8)
        o1x_col_factor = empty((n,), torch.float32)
        o1x_workspace = torch.zeros(((lib.adg_o1x_workspace_bytes(n) + 15) // 16 * 4,), dtype=torch.int32, device=device)
    elif variant == "o0":
        conv_weight = empty((n, k), torch.float16)
        conv_act = empty((m, k), torch.float16)
    elif variant == "o1":
        conv_weight = empty((n, k), torch.int8)
        if m > 64:
            # buffers of the BF16-operand O1 kernel (used while the operands are inside its exact range)
            conv_weight_bf16 = empty((n, k), torch.bfloat16)
            conv_act_bf16 = empty((m, k), torch.bfloat16)
            range_flag = torch.zeros(1, dtype=torch.int32, device=device)
    else:
        conv_weight = empty((lib.adg_o2_tiled_scale_bytes(n, k),), torch.uint8)
        conv_act = empty((m, k // 2), torch.uint8)
        conv_act_sf = empty((m, k // 32), torch.uint8)
        conv_act_sf_tiled = torch.zeros((lib.adg_o2_tiled_scale_bytes(m, k),), dtype=torch.uint8, device=device)

    times = {name: (c_float * repeats)() for name, _ in _STAGE_BITS}
    args = BenchArgs()
    args.variant, args.mode = _VARIANTS[variant], _MODES[mode]
    args.M, args.N, args.K = m, n, k
    args.warmup, args.repeats, args.conversion_inner_repeats = warmup, repeats, conversion_inner_repeats
    args.a_int8, args.a_scale = a_int8.data_ptr(), a_scale.data_ptr()
    args.w_mxfp4, args.w_scale = w_mxfp4.data_ptr(), w_scale.data_ptr()
    args.output = output.data_ptr()
    args.conv_weight = conv_weight.data_ptr()
    args.conv_act = conv_act.data_ptr() if conv_act is not None else None
    args.conv_act_sf = conv_act_sf.data_ptr() if conv_act_sf is not None else None
    args.conv_act_sf_tiled = conv_act_sf_tiled.data_ptr() if conv_act_sf_tiled is not None else None
    args.conv_weight_bf16 = conv_weight_bf16.data_ptr() if conv_weight_bf16 is not None else None
    args.conv_act_bf16 = conv_act_bf16.data_ptr() if conv_act_bf16 is not None else None
    args.range_flag = range_flag.data_ptr() if range_flag is not None else None
    l2_flush = torch.empty((L2_FLUSH_BYTES,), dtype=torch.uint8, device=device) if flush_l2 else None
    args.flags = ((BENCH_FUSE_ACTIVATION if fused else 0) | (BENCH_O1_SPLIT_ACTIVATION if o1_split_activation_stage else 0)
                  | (BENCH_FLUSH_L2 if flush_l2 else 0))
    args.l2_flush = l2_flush.data_ptr() if l2_flush is not None else None
    args.l2_flush_bytes = L2_FLUSH_BYTES if l2_flush is not None else 0
    args.row_counters = row_counters.data_ptr() if row_counters is not None else None
    args.o1x_col_factor = o1x_col_factor.data_ptr() if o1x_col_factor is not None else None
    args.o1x_workspace = o1x_workspace.data_ptr() if o1x_workspace is not None else None
    args.o1x_w_int8 = o1x_w_int8.data_ptr() if o1x_w_int8 is not None else None
    args.t_weight = ctypes.cast(times["weight_conversion"], POINTER(c_float))
    args.t_activation = ctypes.cast(times["activation_conversion"], POINTER(c_float))
    args.t_gemm = ctypes.cast(times["gemm"], POINTER(c_float))
    args.t_total = ctypes.cast(times["total"], POINTER(c_float))
    with torch.cuda.device(device):
        args.stream = torch.cuda.current_stream(device).cuda_stream
        _check(lib.adg_benchmark(ctypes.byref(args)))

    timings = {name: list(times[name]) for name, bit in _STAGE_BITS if args.stages_out & bit}
    if variant == "o0":
        converted_weight, converted_activation = conv_weight, conv_act
    elif variant in ("o1", "o1x"):
        converted_weight, converted_activation = conv_weight, None
    else:
        converted_weight, converted_activation = None, (conv_act, conv_act_sf)
    extra = {}
    if variant == "o1x":
        rows = c_int64(0)
        with torch.cuda.device(device):
            _check(lib.adg_o1x_ineligible_rows(o1x_workspace.data_ptr(), args.stream, ctypes.byref(rows)))
        extra = {"o1x_ineligible_rows": int(rows.value), "o1x_column_factor": o1x_col_factor}
    return {
        **extra,
        "output": output,
        "converted_weight": converted_weight,
        "converted_activation": converted_activation,
        "timings_ms": timings,
        "timing_method": {**_timing_metadata(mode, conversion_inner_repeats),
                          "l2": "flushed before every directly timed iteration" if flush_l2 else "as the previous iteration left it"},
        "kernel": kernel_metadata(variant, m, n, k, o1_bf16=range_flag is not None and int(range_flag.item()) == 0,
                                  fused=fused),
    }


def _run(variant, a_int8, a_scale, w_mxfp4, w_scale, mode):
    # reference adangel_run_o{0,1,2}: one un-warmed repetition plus scalar *_ms keys
    result = benchmark(variant, mode, a_int8, a_scale, w_mxfp4, w_scale, 0, 1, DEFAULT_CONVERSION_INNER_REPEATS)
    timings = result["timings_ms"]
    for stage, key in (("weight_conversion", "weight_conversion_ms"),
                       ("activation_conversion", "activation_conversion_ms"),
                       ("gemm", "gemm_ms"), ("total", "total_ms")):
        result[key] = float(timings[stage][0]) if stage in timings else 0.0
    return result


def run_o0(a_int8, a_scale, w_mxfp4, w_scale, mode):
    return _run("o0", a_int8, a_scale, w_mxfp4, w_scale, mode)


def run_o1(a_int8, a_scale, w_mxfp4, w_scale, mode):
    return _run("o1", a_int8, a_scale, w_mxfp4, w_scale, mode)


def run_o2(a_int8, a_scale, w_mxfp4, w_scale, mode):
    return _run("o2", a_int8, a_scale, w_mxfp4, w_scale, mode)


def run_o1x(a_int8, a_scale, w_mxfp4, w_scale, mode):
    """The exact-integer O1 variant (no reference counterpart; see ``adg_gemm_o1x``)."""
    return _run("o1x", a_int8, a_scale, w_mxfp4, w_scale, mode)


def verify_layout() -> dict:
    passed = c_int(0)
    err = c_float(0.0)
    _check(library().adg_verify_layout(ctypes.byref(passed), ctypes.byref(err)))
    return {"passed": bool(passed.value), "max_abs_error": float(err.value)}
