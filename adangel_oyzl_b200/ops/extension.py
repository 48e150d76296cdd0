"""Native library discovery and strict SM100 capability checks.

Mirrors ``python/adangel/ops/extension.py:19-114`` of the reference with every literal re-targeted
from RTX 5090 / sm_120a to B200 / sm_100a.  The "extension module" is :mod:`._sm100`, a ctypes
binding of ``libadangel_b200.so``; there is no fallback when it is missing.
"""

from __future__ import annotations

import importlib
from dataclasses import dataclass

REQUIRED_CAPABILITY = (10, 0)
REQUIRED_DEVICE_SUBSTRING = "B200"
MIN_TORCH_CUDA = (12, 8)


@dataclass(frozen=True)
class NativeStatus:
    available: bool
    reason: str
    capabilities: dict


def load_native():
    try:
        module = importlib.import_module("adangel_oyzl_b200.ops._sm100")
        module.library()  # dlopen now so that a missing build shows up here
        return module
    except (ImportError, OSError):
        return None


def _environment_problem():
    try:
        import torch
    except ImportError:
        return "PyTorch is not installed"
    cuda = torch.version.cuda
    if cuda is None or tuple(int(x) for x in cuda.split(".")[:2]) < MIN_TORCH_CUDA:
        return f"requires PyTorch built for CUDA >= {MIN_TORCH_CUDA[0]}.{MIN_TORCH_CUDA[1]}, found {cuda}"
    if not torch.cuda.is_available():
        return "CUDA is not available"
    name = torch.cuda.get_device_name(0)
    capability = tuple(torch.cuda.get_device_capability(0))
    if REQUIRED_DEVICE_SUBSTRING not in name or capability != REQUIRED_CAPABILITY:
        return f"requires B200 sm_100, found {name} sm_{capability[0]}{capability[1]}"
    return None


def native_status() -> NativeStatus:
    problem = _environment_problem()
    if problem is not None:
        return NativeStatus(False, problem, {})
    extension = load_native()
    if extension is None:
        return NativeStatus(False, "adangel_oyzl_b200 native library is not built", {})
    capabilities = dict(extension.capabilities())
    required = (
        "o0_fp16_tc",
        "o1_int8_tc",
        "o2_mxf4_block_scale",
        "o2_cutlass_tiled",
        "compiled_sm100a",
    )
    missing = [key for key in required if not capabilities.get(key, False)]
    if missing:
        return NativeStatus(False, f"native extension lacks: {', '.join(missing)}", capabilities)
    return NativeStatus(True, "ready", capabilities)


def require_sm100_extension():
    problem = _environment_problem()
    if problem is not None:
        raise RuntimeError(problem)
    extension = load_native()
    if extension is None:
        raise RuntimeError("adangel_oyzl_b200 native library is not built")
    capabilities = dict(extension.capabilities())
    if not capabilities.get("compiled_sm100a", False):
        raise RuntimeError("extension was not compiled for sm_100a")
    return extension


def require_native():
    status = native_status()
    if not status.available:
        raise RuntimeError(f"formal SM100 backend unavailable: {status.reason}")
    return load_native()


def require_variant(variant: str):
    """Require only the production capability needed by one public variant call."""
    extension = require_sm100_extension()
    capabilities = dict(extension.capabilities())
    required = {
        "o0": ("o0_fp16_tc",),
        "o1": ("o1_int8_tc",),
        "o2": ("o2_mxf4_block_scale", "o2_cutlass_tiled"),
        "o1x": ("o1_int8_tc",),  # the exact-integer O1 variant of this build; only ever requested by name
    }
    if variant not in required:
        raise ValueError(f"unknown variant: {variant}")
    missing = [key for key in required[variant] if not capabilities.get(key, False)]
    if missing:
        raise RuntimeError(
            f"formal SM100 {variant.upper()} backend unavailable: native extension lacks: "
            f"{', '.join(missing)}"
        )
    return extension
