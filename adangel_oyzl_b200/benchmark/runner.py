"""Interleaved O0/O1/O2 experiment runner writing ``results.jsonl`` records of schema version 2.

Follows the reference's formal runner (``python/adangel/benchmark/runner.py:18-207``): for every
sample, every mode and every variant (variants interleaved inside a mode) one native benchmark call,
payload validation, per-stage statistics with the CV gate, byte and equivalent-FLOP accounting, and
the FP64 MSE of every variant's ``compute_only`` output against O0's.  Two differences: samples are
seeded synthetic inputs instead of prepared Llama-2 traces (no model or dataset is available
offline), and a config may list several ``matrix.shapes``.  Records keep every reference key;
``roofline`` and ``bytes_moved_fused`` are additions that the analysis ignores.
"""

from __future__ import annotations

import json
from pathlib import Path

import yaml

from ..ops.dispatch import benchmark_variant
from ..ops.extension import require_native
from .metadata import write_environment
from .metrics import mse_fp64, summarize_samples

NOMINAL_TFLOPS = {"o0": 2250.0, "o1": 4500.0, "o1x": 4500.0, "o2": 9000.0}  # dense FP16 / INT8 / FP4 on B200
NOMINAL_HBM_GBS = 8000.0


def _throughput_tflops(m: int, n: int, k: int, ms: float) -> float:
    return (2.0 * m * n * k) / ms / 1.0e9 if ms > 0 else 0.0


DECODE_MAX_M = 64  # activations up to this many rows take the weight-streaming decode kernels


def _conversion_bytes(variant: str, stage: str, m: int, n: int, k: int) -> int:
    """Bytes each conversion stage moves, with the reference's accounting (runner.py:22-37)."""
    natural_sfa = m * (k // 32)
    natural_sfb = n * (k // 32)
    sizes = {
        ("o0", "weight_conversion"): n * k // 2 + n * (k // 32) + 2 * n * k,
        ("o0", "activation_conversion"): m * k + 4 * m + 2 * m * k,
        ("o1", "weight_conversion"): n * k // 2 + n * k,
        ("o1x", "weight_conversion"): 2 * (n * k // 2 + n * k) + n * (k // 32),  # both INT8 images, scales read once
        ("o2", "activation_conversion"): m * k + 4 * m + m * k // 2 + 3 * natural_sfa,
        ("o2", "weight_conversion"): 2 * natural_sfb,
    }
    if stage == "gemm" and m <= DECODE_MAX_M:
        # decode shapes are weight-streaming: the GEMM itself is reported in GB/s (W once, A, scales, Y)
        sizes[("o1", "gemm")] = n * k + natural_sfb + m * k + 4 * m + 4 * m * n
        sizes[("o2", "gemm")] = n * k // 2 + natural_sfb + m * k // 2 + natural_sfa + 4 * m * n
    return sizes.get((variant, stage), 0)


def _fused_conversion_bytes(variant: str, stage: str, m: int, n: int, k: int, o1_bf16: bool = False) -> int:
    """What the conversion kernels of this build actually move: the fused O2 activation kernel (one
    natural and one tiled scale write, no separate re-layout pass) and, when O1 runs on BF16 operands,
    its activation conversion and the second (BF16) form of its weight; equal to the reference figure
    for the other stages."""
    if (variant, stage) == ("o2", "activation_conversion"):
        return m * k + 4 * m + m * k // 2 + 2 * m * (k // 32)
    if variant == "o1" and o1_bf16 and stage == "activation_conversion":
        return m * k + 4 * m + 2 * m * k
    if variant == "o1" and o1_bf16 and stage == "weight_conversion":
        return (n * k // 2 + n * k) + (n * k // 2 + n * (k // 32) + 2 * n * k)
    return _conversion_bytes(variant, stage, m, n, k)


def _summarize_timings(timings: dict, max_cv: float):
    summaries = {stage: summarize_samples(values) for stage, values in timings.items() if values}
    stable = all(float(item["cv_percent"]) < max_cv for item in summaries.values())
    return summaries, stable


def _validate_benchmark_payload(payload: dict, repeats: int, mode: str, conversion_inner_repeats: int) -> None:
    if "output" not in payload or "timings_ms" not in payload:
        raise RuntimeError("native benchmark must return output and timings_ms")
    allowed = {"weight_conversion", "activation_conversion", "gemm", "total"}
    unknown = set(payload["timings_ms"]) - allowed
    if unknown:
        raise RuntimeError(f"unknown native timing stages: {sorted(unknown)}")
    for name, values in payload["timings_ms"].items():
        if len(values) != repeats:
            raise RuntimeError(f"stage {name} returned {len(values)} samples, expected {repeats}")
    timing_method = payload.get("timing_method")
    if not isinstance(timing_method, dict):
        raise RuntimeError("native benchmark must return timing_method metadata")
    if timing_method.get("strategy") != "conversion_amortized_end_to_end_direct":
        raise RuntimeError("native benchmark returned an unexpected timing strategy")
    if int(timing_method.get("conversion_inner_repeats", 0)) != conversion_inner_repeats:
        raise RuntimeError("native benchmark conversion_inner_repeats does not match config")
    expected_total_method = "batched_cuda_event_average" if mode == "conversion_only" else "direct_single_path"
    if timing_method.get("mode_total_timing") != expected_total_method:
        raise RuntimeError(f"{mode}: native benchmark returned the wrong total timing method")


def _shapes(config: dict) -> list[tuple[int, int, int]]:
    matrix = config["matrix"]
    if "shapes" in matrix:
        return [tuple(int(x) for x in shape) for shape in matrix["shapes"]]
    return [(int(matrix["m"]), int(matrix["n"]), int(matrix["k"]))]


def _roofline(variant: str, summaries: dict, m: int, n: int, k: int, o1_bf16: bool = False) -> dict:
    out = {}
    gemm = summaries.get("gemm")
    if gemm and gemm["median_ms"] > 0:
        tf = _throughput_tflops(m, n, k, gemm["median_ms"])
        out["gemm"] = {"bound": "tensor", "achieved_tflops": tf, "nominal_peak_tflops": NOMINAL_TFLOPS[variant],
                       "fraction_of_nominal": tf / NOMINAL_TFLOPS[variant]}
    for stage in ("weight_conversion", "activation_conversion"):
        stats = summaries.get(stage)
        nbytes = _fused_conversion_bytes(variant, stage, m, n, k, o1_bf16)
        if stats and nbytes and stats["median_ms"] > 0:
            gbs = nbytes / stats["median_ms"] / 1.0e6
            out[stage] = {"bound": "hbm", "achieved_gbs": gbs, "nominal_peak_gbs": NOMINAL_HBM_GBS,
                          "fraction_of_nominal": gbs / NOMINAL_HBM_GBS}
    return out


def _iter_samples(config, n_samples, device, prepared_dir, formal):
    """The experiment's samples: loaded from a prepared directory (manifest order, hashes checked)
    or generated from the seeded synthetic distribution, ``n_samples`` per configured shape."""
    if prepared_dir is not None:
        from ..trace.storage import load_manifest, load_prepared

        prepared_dir = Path(prepared_dir)
        manifest = load_manifest(prepared_dir, formal=formal)
        for record in manifest["samples"][:n_samples]:
            yield load_prepared(prepared_dir / record["file"], device=device, expected_sha256=record["sha256"])
        return
    from ..synthetic import canonical_inputs

    seed = int(config["experiment"]["seed"])
    for m, n, k in _shapes(config):
        for sample_index in range(n_samples):
            yield canonical_inputs(m, n, k, seed=seed + sample_index, device=device,
                                   sample_id=f"synthetic_{m}x{n}x{k}_s{sample_index:02d}")


def run_experiment(config_path, output_dir, *, sample_limit=None, warmup_override=None, repeats_override=None,
                   device="cuda", prepared_dir=None) -> Path:
    import torch

    require_native()
    config_path, output_dir = Path(config_path), Path(output_dir)
    config = yaml.safe_load(config_path.read_text(encoding="utf-8"))
    if config["backend"]["required"] != "native":
        raise ValueError("the runner requires backend.required=native")
    timing = config["timing"]
    warmup = int(warmup_override if warmup_override is not None else timing["warmup"])
    repeats = int(repeats_override if repeats_override is not None else timing["repeats"])
    conversion_inner_repeats = int(timing["conversion_inner_repeats"])
    if warmup < 0 or repeats <= 0 or conversion_inner_repeats <= 1:
        raise ValueError("warmup must be non-negative, repeats must be positive, and "
                         "conversion_inner_repeats must exceed one")
    n_samples = int(config["data"]["samples"])
    if prepared_dir is not None:
        # a prepared directory brings its own sample list
        from ..trace.storage import load_manifest

        n_samples = len(load_manifest(Path(prepared_dir), formal=bool(config["experiment"].get("formal", False)))["samples"])
    if sample_limit is not None:
        if not 1 <= sample_limit <= n_samples:
            raise ValueError(f"samples must be in [1,{n_samples}]")
        n_samples = sample_limit
    if output_dir.exists() and any(output_dir.iterdir()):
        raise FileExistsError(f"refusing to overwrite non-empty run directory: {output_dir}")
    output_dir.mkdir(parents=True, exist_ok=True)
    resolved = dict(config)
    resolved["timing"] = {**timing, "warmup": warmup, "repeats": repeats}
    (output_dir / "config.yaml").write_text(yaml.safe_dump(resolved, sort_keys=False), encoding="utf-8")
    write_environment(output_dir / "environment.json")

    max_cv = float(timing["max_cv_percent"])
    flush_l2 = bool(timing.get("flush_l2", False))  # decode shapes: operands from HBM, not from a warm L2
    modes = list(config["modes"])
    variants = list(config["variants"])
    formal = bool(config["experiment"].get("formal", False))
    with (output_dir / "results.jsonl").open("w", encoding="utf-8") as stream:
        for inputs in _iter_samples(config, n_samples, device, prepared_dir, formal):
            shape = m, n, k = inputs.shape
            records = []
            # variants are interleaved inside each mode to reduce temperature/boost drift
            for mode in modes:
                for variant in variants:
                    payload = benchmark_variant(inputs, variant, mode, warmup, repeats, backend="native",
                                                conversion_inner_repeats=conversion_inner_repeats,
                                                formal=formal and shape == (4096, 4096, 4096), flush_l2=flush_l2)
                    _validate_benchmark_payload(payload, repeats, mode, conversion_inner_repeats)
                    summaries, stable = _summarize_timings(payload["timings_ms"], max_cv)
                    for stage, stats in summaries.items():
                        byte_count = _conversion_bytes(variant, stage, m, n, k)
                        stats["bytes_moved"] = byte_count
                        stats["bytes_moved_fused"] = _fused_conversion_bytes(variant, stage, m, n, k)
                        stats["throughput_gbps"] = (byte_count / float(stats["median_ms"]) / 1.0e6
                                                    if byte_count and float(stats["median_ms"]) > 0 else 0.0)
                    gemm_median = summaries.get("gemm", {}).get("median_ms", 0.0)
                    record = {
                        "schema_version": 2,
                        "sample_id": inputs.sample_id,
                        "variant": variant,
                        "mode": mode,
                        "shape": [m, n, k],
                        "timings_ms": payload["timings_ms"],
                        "summary": summaries,
                        "equivalent_tflops": _throughput_tflops(m, n, k, float(gemm_median)),
                        "mse_vs_o0": None,
                        "kernel": payload.get("kernel"),
                        "timing_method": payload.get("timing_method"),
                        "l2_flushed": flush_l2,
                        "stable_cv": stable,
                        "valid": stable,
                        "roofline": _roofline(variant, summaries, m, n, k,
                                              o1_bf16=(payload.get("kernel") or {}).get("kernel_symbol") == "gemm_o1_bf16_kernel"),
                    }
                    records.append((record, payload["output"] if mode == "compute_only" else None))
                    del payload
            outputs = {r["variant"]: out for r, out in records if r["mode"] == "compute_only"}
            mse = {}
            if "o0" in outputs:
                reference = outputs["o0"]
                if not torch.isfinite(reference).all():
                    raise RuntimeError(f"{inputs.sample_id}: O0 output contains NaN/Inf")
                mse = {name: mse_fp64(out, reference) for name, out in outputs.items()}
            for record, _ in records:
                record["mse_vs_o0"] = mse.get(record["variant"])
                stream.write(json.dumps(record, ensure_ascii=False) + "\n")
                stream.flush()
            del inputs, records, outputs
            torch.cuda.empty_cache()
    return output_dir
