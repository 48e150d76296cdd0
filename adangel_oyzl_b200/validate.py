"""Acceptance check of one variant on the device: the counterpart of the reference's
``scripts/validate_o{0,1,2}.py`` (e.g. ``scripts/validate_o1.py:120-200``).

For one variant and shape it runs the four timing modes through the ops surface and checks what those
scripts check that needs no second implementation: the stage set of every mode, the timing-method
metadata, finite FP32 outputs that are bit-identical across the four modes, the kernel metadata, and --
at the formal 4096^3 shape -- the performance gate: compute-only GEMM median below ``max_compute_ms`` and
its coefficient of variation below ``max_cv_percent`` (the reference gates at 3 %).  Agreement with the
semantic reference is the business of the test-suite, which passes the expected output in
(``expected_output``); this module never computes a reference result itself.
"""

from __future__ import annotations

from .benchmark.metrics import summarize_samples

EXPECTED_STAGES = {
    "o0": {"conversion_only": {"weight_conversion", "activation_conversion", "total"}, "compute_only": {"gemm", "total"},
           "cold": {"weight_conversion", "activation_conversion", "gemm", "total"},
           "steady_state": {"activation_conversion", "gemm", "total"}},
    "o1": {"conversion_only": {"weight_conversion", "total"}, "compute_only": {"gemm", "total"},
           "cold": {"weight_conversion", "gemm", "total"}, "steady_state": {"gemm", "total"}},
}
EXPECTED_STAGES["o2"] = EXPECTED_STAGES["o0"]
EXPECTED_STAGES["o1x"] = EXPECTED_STAGES["o1"]
# generous ceilings for the 4096^3 compute-only GEMM on a B200 (about 1.5x the measured medians)
DEFAULT_MAX_COMPUTE_MS = {"o0": 0.16, "o1": 0.50, "o1x": 0.12, "o2": 0.07}


def validate_variant(variant: str, inputs, *, warmup: int = 10, repeats: int = 50, conversion_inner_repeats: int = 100,
                     max_compute_ms: float | None = None, max_cv_percent: float = 3.0, expected_output=None,
                     rtol: float = 1e-3, atol: float = 1e-3) -> dict:
    """Returns a report dictionary with ``passed`` and ``violations``; raises only on contract breaks that the
    reference's scripts raise on too (wrong stage set, wrong timing metadata)."""
    import torch

    from .ops.extension import require_variant

    if variant not in EXPECTED_STAGES:
        raise ValueError(f"unknown variant: {variant}")
    native = require_variant(variant)
    shape = inputs.shape
    modes, methods, outputs, kernel = {}, {}, {}, None
    for mode, stages in EXPECTED_STAGES[variant].items():
        payload = native.benchmark(variant, mode, inputs.A_int8, inputs.A_scale, inputs.W_mxfp4, inputs.W_scale,
                                   warmup, repeats, conversion_inner_repeats)
        torch.cuda.synchronize()
        timings = dict(payload["timings_ms"])
        if set(timings) != stages:
            raise RuntimeError(f"{mode}: expected stages {sorted(stages)}, got {sorted(timings)}")
        method = dict(payload["timing_method"])
        if method.get("strategy") != "conversion_amortized_end_to_end_direct" or \
                method.get("mode_total_timing") != ("batched_cuda_event_average" if mode == "conversion_only" else "direct_single_path"):
            raise RuntimeError(f"{mode}: unexpected timing method {method}")
        methods[mode] = method
        modes[mode] = {stage: summarize_samples(values) for stage, values in timings.items()}
        outputs[mode] = payload["output"]
        kernel = dict(payload["kernel"]) if mode == "compute_only" else kernel
    violations = []
    first = outputs["compute_only"]
    if first.dtype != torch.float32 or not bool(torch.isfinite(first).all()):
        violations.append("compute_only output is not finite FP32")
    for mode, out in outputs.items():
        if not torch.equal(out, first):
            violations.append(f"{mode} output differs from the compute_only output")
    max_abs_error = None
    if expected_output is not None:
        max_abs_error = float((first - expected_output.to(first.device)).abs().max().item())
        if not torch.allclose(first, expected_output.to(first.device), rtol=rtol, atol=atol):
            violations.append(f"output outside rtol={rtol} atol={atol} of the expected output (max abs error {max_abs_error:.3e})")
    for key, value in (("tensor_core", True), ("data_movement", "TMA"), ("global_partial_buffer", False),
                       ("output_stores_per_element", 1), ("group_size", 32)):
        if kernel.get(key) != value:
            violations.append(f"kernel metadata {key}: expected {value!r}, got {kernel.get(key)!r}")
    formal = tuple(shape) == (4096, 4096, 4096)
    limit = DEFAULT_MAX_COMPUTE_MS[variant] if max_compute_ms is None else max_compute_ms
    compute = modes["compute_only"]["gemm"]
    if formal and compute["median_ms"] > limit:
        violations.append(f"compute-only median {compute['median_ms']:.6f} ms exceeds {limit:.6f} ms")
    if formal and compute["cv_percent"] >= max_cv_percent:
        violations.append(f"compute-only CV {compute['cv_percent']:.3f}% must be below {max_cv_percent:.3f}%")
    return {
        "passed": not violations,
        "variant": variant,
        "shape": list(shape),
        "max_abs_error": max_abs_error,
        "kernel": kernel,
        "timing_method_by_mode": methods,
        "modes": modes,
        "performance_gate": {"applied": formal, "max_compute_ms": limit, "max_cv_percent": max_cv_percent},
        "violations": violations,
    }
