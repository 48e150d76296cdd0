"""On-disk format of prepared samples: one ``<sample_id>.pt`` per sample plus ``manifest.json``.

Same format, field names and checks as the reference (``python/adangel/trace/storage.py:11-119``),
so that a directory written by either side loads on the other: manifest version 2, format tag
``adangel-prepared-mxfp4-k32``, a SHA-256 per sample file, and for formal experiments the 24
configured 4096^3 samples.  Non-formal manifests (the other benchmark shapes, synthetic samples)
only need well-formed sample records.
"""

from __future__ import annotations

import hashlib
import json
import re
from pathlib import Path

from ..schema import PreparedInputs, validate_prepared

MANIFEST_VERSION = 2
PREPARED_FORMAT = "adangel-prepared-mxfp4-k32"
FORMAL_SHAPE = [4096, 4096, 4096]
FORMAL_LAYERS = [0, 6, 12, 18, 24, 31]
FORMAL_PROJECTIONS = ["q_proj", "k_proj", "v_proj", "o_proj"]
FORMAL_DTYPES = {"A_int8": "torch.int8", "A_scale": "torch.float32", "W_mxfp4": "torch.uint8", "W_scale": "torch.uint8"}
_SAMPLE_FIELDS = {"sample_id", "file", "sha256", "shape", "layer", "projection"}


def sha256_file(path: Path) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as stream:
        while True:
            chunk = stream.read(1 << 20)
            if not chunk:
                break
            digest.update(chunk)
    return digest.hexdigest()


def save_prepared(inputs: PreparedInputs, output_dir: Path) -> dict:
    """Write one sample (tensors moved to host memory) and return its manifest record."""
    import torch

    validate_prepared(inputs)
    output_dir = Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    path = output_dir / f"{inputs.sample_id}.pt"
    payload = {"sample_id": inputs.sample_id}
    for name in ("A_int8", "A_scale", "W_mxfp4", "W_scale"):
        payload[name] = getattr(inputs, name).cpu()
    payload["shape"] = list(inputs.shape)
    torch.save(payload, path)
    return {"sample_id": inputs.sample_id, "file": path.name, "sha256": sha256_file(path), "shape": list(inputs.shape)}


def load_prepared(path: Path, device: str = "cuda", expected_sha256: str | None = None) -> PreparedInputs:
    """Load and validate one sample; ``expected_sha256`` (from the manifest) is checked first."""
    import torch

    path = Path(path)
    if expected_sha256 is not None and sha256_file(path) != expected_sha256:
        raise ValueError(f"{path}: SHA-256 does not match the manifest")
    record = torch.load(path, map_location=device, weights_only=True)
    inputs = PreparedInputs(record["sample_id"], record["A_int8"], record["A_scale"], record["W_mxfp4"], record["W_scale"])
    validate_prepared(inputs)
    if list(inputs.shape) != list(record.get("shape", [])):
        raise ValueError(f"{path}: embedded shape does not match tensors")
    return inputs


def validate_manifest(manifest: dict, *, formal: bool = False) -> None:
    if manifest.get("version") != MANIFEST_VERSION or manifest.get("format") != PREPARED_FORMAT:
        raise ValueError("unsupported prepared manifest version/format")
    samples = manifest.get("samples")
    if not isinstance(samples, list) or not samples:
        raise ValueError("manifest samples must be a non-empty list")
    seen_ids: set = set()
    seen_files: set = set()
    for sample in samples:
        if not isinstance(sample, dict) or not _SAMPLE_FIELDS.issubset(sample):
            raise ValueError("manifest sample is missing required fields")
        sample_id, filename = sample["sample_id"], sample["file"]
        if sample_id in seen_ids or filename in seen_files:
            raise ValueError("manifest contains duplicate sample_id or filename")
        if filename != f"{sample_id}.pt" or Path(filename).name != filename:
            raise ValueError(f"unsafe or mismatched sample filename: {filename}")
        if not re.fullmatch(r"[0-9a-f]{64}", str(sample["sha256"])):
            raise ValueError(f"invalid SHA-256 for {sample_id}")
        seen_ids.add(sample_id)
        seen_files.add(filename)
    if not formal:
        return
    if manifest.get("matrix_shape") != FORMAL_SHAPE:
        raise ValueError(f"formal manifest must use shape {FORMAL_SHAPE}")
    if any(sample["shape"] != FORMAL_SHAPE for sample in samples):
        raise ValueError("formal sample shape mismatch")
    if manifest.get("dtypes") != FORMAL_DTYPES:
        raise ValueError("formal manifest dtype contract mismatch")
    quantization = manifest.get("quantization", {})
    if quantization.get("activation") != "int8_symmetric_per_row" or quantization.get("weight") != "mxfp4_e2m1_ue8m0_k32":
        raise ValueError("formal manifest quantization contract mismatch")
    trace = manifest.get("trace", {})
    if trace.get("layers") != FORMAL_LAYERS or trace.get("projections") != FORMAL_PROJECTIONS:
        raise ValueError("formal trace selection mismatch")
    expected_ids = {f"layer_{layer:02d}_{projection}" for layer in FORMAL_LAYERS for projection in FORMAL_PROJECTIONS}
    if len(samples) != len(expected_ids) or seen_ids != expected_ids:
        raise ValueError("formal manifest must contain exactly the 24 configured samples")


def write_manifest(output_dir: Path, samples: list, metadata: dict, *, formal: bool = True) -> dict:
    manifest = {"version": MANIFEST_VERSION, "format": PREPARED_FORMAT, **metadata, "samples": samples}
    validate_manifest(manifest, formal=formal)
    (Path(output_dir) / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n", encoding="utf-8")
    return manifest


def load_manifest(directory: Path, *, formal: bool = False) -> dict:
    manifest = json.loads((Path(directory) / "manifest.json").read_text(encoding="utf-8"))
    validate_manifest(manifest, formal=formal)
    return manifest
