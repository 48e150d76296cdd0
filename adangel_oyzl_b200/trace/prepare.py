"""Turn floating-point activations / weights into prepared samples, quantizing on the GPU.

``prepare_trace`` is the counterpart of the reference's ``prepare_trace``
(``python/adangel/trace/prepare.py:82-140``): it reads the 24 raw FP16 sample files of an external
prefill trace, quantizes each (per-row INT8 activations, MXFP4 weights) and writes the prepared
directory with its formal manifest.  The two quantizers run as CUDA kernels
(``csrc/prepare.cu``) instead of torch CPU ops; their results are bit-identical to the CPU functions.
What this module does NOT re-implement is the deep validation of the raw trace's provenance
(collector environment, tokenisation hashes: ``trace/raw.py`` of the reference): the raw manifest is
required and its hash and selected fields are recorded, nothing more.

``prepare_synthetic`` writes the seeded synthetic samples of the other benchmark shapes in the same
on-disk format (non-formal manifest).
"""

from __future__ import annotations

import json
from pathlib import Path

from ..schema import PreparedInputs
from .storage import (FORMAL_DTYPES, FORMAL_LAYERS, FORMAL_PROJECTIONS, FORMAL_SHAPE, save_prepared, sha256_file,
                      write_manifest)

RAW_MANIFEST_NAME = "trace_manifest.json"
_QUANTIZATION = {"activation": "int8_symmetric_per_row", "weight": "mxfp4_e2m1_ue8m0_k32", "rounding": "round_ties_to_even"}


def _config(value):
    if isinstance(value, dict):
        return value
    import yaml

    return yaml.safe_load(Path(value).read_text(encoding="utf-8"))


def validate_configs(experiment: dict, trace: dict):
    """The experiment / trace configuration contract of the formal preparation
    (reference ``prepare.py:22-34`` and ``raw.py:44-60``)."""
    matrix = experiment.get("matrix", {})
    if [matrix.get("m"), matrix.get("n"), matrix.get("k")] != FORMAL_SHAPE:
        raise ValueError("trace preparation requires M=N=K=4096")
    quantization = experiment.get("quantization", {})
    if quantization.get("activation", {}).get("format") != "int8_symmetric_per_row":
        raise ValueError("activation quantization must be int8_symmetric_per_row")
    weight = quantization.get("weight", {})
    if weight.get("format") != "mxfp4_e2m1_ue8m0" or weight.get("group_size") != 32:
        raise ValueError("weight quantization must be MXFP4 E2M1/UE8M0 K32")
    layers = [int(v) for v in trace.get("layers", [])]
    projections = list(trace.get("projections", []))
    if layers != FORMAL_LAYERS:
        raise ValueError(f"trace layers must be {FORMAL_LAYERS}")
    if projections != FORMAL_PROJECTIONS:
        raise ValueError(f"trace projections must be {FORMAL_PROJECTIONS}")
    if trace.get("batch_size") != 1 or int(trace.get("sequence_length", 0)) != 4096:
        raise ValueError("formal trace requires batch=1 and sequence_length=4096")
    if str(trace.get("dtype", "")).lower() not in {"fp16", "float16"}:
        raise ValueError("formal trace dtype must be fp16")
    return layers, projections


def load_raw_sample(path: Path, layer: int, projection: str):
    """One raw trace file: identity, dtype, shape, contiguity and finiteness checks
    (reference ``prepare.py:37-58``)."""
    import torch

    raw = torch.load(path, map_location="cpu", weights_only=True)
    required = {"sample_id", "layer", "projection", "activation_fp16", "weight_fp16"}
    if not isinstance(raw, dict) or not required.issubset(raw):
        raise ValueError(f"{path.name}: missing required raw trace fields")
    sample_id = f"layer_{layer:02d}_{projection}"
    if raw["sample_id"] != sample_id or raw["layer"] != layer or raw["projection"] != projection:
        raise ValueError(f"{path.name}: sample metadata does not match its configured identity")
    for name in ("activation_fp16", "weight_fp16"):
        tensor = raw[name]
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{path.name}: {name} must be a torch.Tensor")
        if tuple(tensor.shape) != (4096, 4096) or tensor.dtype != torch.float16:
            raise ValueError(f"{path.name}: {name} must be [4096,4096] torch.float16")
        if not tensor.is_contiguous():
            raise ValueError(f"{path.name}: {name} must be contiguous")
        if not torch.isfinite(tensor).all():
            raise ValueError(f"{path.name}: {name} contains NaN/Inf")
    return raw


def quantize_sample(sample_id: str, activation, weight, device="cuda") -> PreparedInputs:
    """Float activation [M,K] and weight [N,K] (float32 or float16, any device) -> prepared sample
    on ``device``, quantized by the CUDA kernels."""
    from .. import kernels

    a = activation.to(device).contiguous()
    w = weight.to(device).contiguous()
    a_int8, a_scale = kernels.quantize_int8_per_row(a)
    w_mxfp4, w_scale = kernels.quantize_mxfp4(w)
    return PreparedInputs(sample_id, a_int8, a_scale, w_mxfp4, w_scale)


def prepare_trace(input_dir, output_dir, experiment_config, trace_config, device="cuda") -> list:
    input_dir, output_dir = Path(input_dir), Path(output_dir)
    layers, projections = validate_configs(_config(experiment_config), _config(trace_config))
    if output_dir.exists() and any(output_dir.iterdir()):
        raise FileExistsError(f"refusing to overwrite non-empty prepared directory: {output_dir}")
    raw_manifest_path = input_dir / RAW_MANIFEST_NAME
    if not raw_manifest_path.is_file():
        raise FileNotFoundError(f"{raw_manifest_path} is required (provenance of the raw trace)")
    raw_manifest = json.loads(raw_manifest_path.read_text(encoding="utf-8"))
    expected = {f"layer_{layer:02d}_{projection}.pt": (layer, projection) for layer in layers for projection in projections}
    missing = [name for name in expected if not (input_dir / name).is_file()]
    if missing:
        raise FileNotFoundError(f"raw trace is missing {len(missing)} sample file(s), first: {missing[0]}")

    records = []
    for filename, (layer, projection) in expected.items():
        raw = load_raw_sample(input_dir / filename, layer, projection)
        prepared = quantize_sample(raw["sample_id"], raw["activation_fp16"], raw["weight_fp16"], device)
        record = save_prepared(prepared, output_dir)
        record.update({"layer": layer, "projection": projection})
        records.append(record)
    write_manifest(output_dir, records, {
        "matrix_shape": FORMAL_SHAPE,
        "dtypes": FORMAL_DTYPES,
        "quantization": dict(_QUANTIZATION, implementation="CUDA kernels quantize_int8_rows / quantize_mxfp4 (exact block exponent)"),
        "trace": {"source": "external_fp16_prefill_trace", "batch_size": 1, "valid_tokens": 4096,
                  "layers": layers, "projections": projections},
        "source_trace": {"manifest_file": RAW_MANIFEST_NAME, "manifest_sha256": sha256_file(raw_manifest_path),
                         "format": raw_manifest.get("format"), "dataset": raw_manifest.get("dataset"),
                         "model": raw_manifest.get("model")},
    }, formal=True)
    return records


def prepare_synthetic(shapes, output_dir, seed=None, device="cuda") -> list:
    """Seeded synthetic samples (one per shape) in the prepared on-disk format; the manifest is
    non-formal and says so."""
    from .. import synthetic

    output_dir = Path(output_dir)
    if output_dir.exists() and any(output_dir.iterdir()):
        raise FileExistsError(f"refusing to overwrite non-empty prepared directory: {output_dir}")
    base_seed = synthetic.CANONICAL_SEED if seed is None else int(seed)
    records = []
    for index, (m, n, k) in enumerate(shapes):
        a, w = synthetic.canonical_floats(int(m), int(n), int(k), base_seed + index)
        sample_id = f"synthetic_{index:02d}_{m}x{n}x{k}"
        record = save_prepared(quantize_sample(sample_id, a, w, device), output_dir)
        record.update({"layer": index, "projection": "synthetic"})
        records.append(record)
    write_manifest(output_dir, records, {
        "dtypes": FORMAL_DTYPES,
        "quantization": dict(_QUANTIZATION),
        "trace": {"source": "synthetic_canonical", "seed": base_seed,
                  "activation": "N(0,1), 0.5% of K channels x20", "weight": "N(0,0.02)"},
    }, formal=False)
    return records
