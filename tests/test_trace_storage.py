"""Prepared-sample storage and manifest contract (CPU).  Mirrors the cases of the reference's
tests/unit/test_manifest_contract.py: well-formed records, duplicate / unsafe names, hash format,
the formal 24-sample selection, and a save -> load round trip with hash verification."""

import copy
import json

import pytest
import torch

from adangel_oyzl_b200 import synthetic
from adangel_oyzl_b200.trace import storage
from adangel_oyzl_b200.trace.prepare import load_raw_sample, validate_configs


def _formal_manifest():
    samples = [{"sample_id": f"layer_{layer:02d}_{proj}", "file": f"layer_{layer:02d}_{proj}.pt", "sha256": "0" * 64,
                "shape": [4096, 4096, 4096], "layer": layer, "projection": proj}
               for layer in storage.FORMAL_LAYERS for proj in storage.FORMAL_PROJECTIONS]
    return {"version": 2, "format": storage.PREPARED_FORMAT, "matrix_shape": [4096, 4096, 4096],
            "dtypes": dict(storage.FORMAL_DTYPES),
            "quantization": {"activation": "int8_symmetric_per_row", "weight": "mxfp4_e2m1_ue8m0_k32"},
            "trace": {"layers": list(storage.FORMAL_LAYERS), "projections": list(storage.FORMAL_PROJECTIONS)},
            "samples": samples}


def test_formal_manifest_accepted_and_rejections():
    good = _formal_manifest()
    storage.validate_manifest(good, formal=True)
    for mutate, message in (
        (lambda m: m.update(version=1), "unsupported prepared manifest"),
        (lambda m: m.update(samples=[]), "non-empty list"),
        (lambda m: m["samples"][0].pop("sha256"), "missing required fields"),
        (lambda m: m["samples"][1].update(sample_id=m["samples"][0]["sample_id"]), "duplicate"),
        (lambda m: m["samples"][0].update(file="../evil.pt"), "unsafe or mismatched"),
        (lambda m: m["samples"][0].update(sha256="xyz"), "invalid SHA-256"),
        (lambda m: m.update(matrix_shape=[128, 128, 128]), "formal manifest must use shape"),
        (lambda m: m["samples"][0].update(shape=[1, 2, 3]), "formal sample shape mismatch"),
        (lambda m: m["dtypes"].update(A_int8="torch.int16"), "dtype contract"),
        (lambda m: m["quantization"].update(weight="nvfp4"), "quantization contract"),
        (lambda m: m["trace"].update(layers=[0, 1]), "trace selection"),
        (lambda m: m["samples"].pop(), "exactly the 24"),
    ):
        bad = copy.deepcopy(good)
        mutate(bad)
        with pytest.raises(ValueError, match=message):
            storage.validate_manifest(bad, formal=True)
    # the same structural errors are caught for non-formal manifests, the formal-only ones are not
    relaxed = copy.deepcopy(good)
    relaxed["matrix_shape"] = [128, 128, 128]
    storage.validate_manifest(relaxed, formal=False)


def test_save_load_round_trip_with_hash(tmp_path):
    sample = synthetic.canonical_inputs(64, 96, 128, seed=5, sample_id="layer_00_q_proj")
    record = storage.save_prepared(sample, tmp_path)
    assert record["file"] == "layer_00_q_proj.pt" and record["shape"] == [64, 96, 128]
    assert record["sha256"] == storage.sha256_file(tmp_path / record["file"])
    loaded = storage.load_prepared(tmp_path / record["file"], device="cpu", expected_sha256=record["sha256"])
    for name in ("A_int8", "A_scale", "W_mxfp4", "W_scale"):
        assert torch.equal(getattr(loaded, name), getattr(sample, name))
    with pytest.raises(ValueError, match="SHA-256 does not match"):
        storage.load_prepared(tmp_path / record["file"], device="cpu", expected_sha256="f" * 64)
    record.update(layer=0, projection="q_proj")
    manifest = storage.write_manifest(tmp_path, [record], {"trace": {"source": "test"}}, formal=False)
    assert json.loads((tmp_path / "manifest.json").read_text())["samples"] == manifest["samples"]
    assert storage.load_manifest(tmp_path)["format"] == storage.PREPARED_FORMAT
    with pytest.raises(ValueError):
        storage.write_manifest(tmp_path, [record], {}, formal=True)  # one sample is not a formal set


def test_save_rejects_malformed_sample(tmp_path):
    sample = synthetic.canonical_inputs(64, 96, 128, seed=5)
    bad = type(sample)(sample.sample_id, sample.A_int8, sample.A_scale[:-1].contiguous(), sample.W_mxfp4, sample.W_scale)
    with pytest.raises(ValueError, match="A_scale"):
        storage.save_prepared(bad, tmp_path)


def test_prepare_config_and_raw_sample_checks(tmp_path):
    experiment = {"matrix": {"m": 4096, "n": 4096, "k": 4096},
                  "quantization": {"activation": {"format": "int8_symmetric_per_row"},
                                   "weight": {"format": "mxfp4_e2m1_ue8m0", "group_size": 32}}}
    trace = {"layers": [0, 6, 12, 18, 24, 31], "projections": ["q_proj", "k_proj", "v_proj", "o_proj"],
             "batch_size": 1, "sequence_length": 4096, "dtype": "fp16"}
    assert validate_configs(experiment, trace) == (trace["layers"], trace["projections"])
    with pytest.raises(ValueError, match="M=N=K=4096"):
        validate_configs({**experiment, "matrix": {"m": 1, "n": 2, "k": 3}}, trace)
    with pytest.raises(ValueError, match="trace layers"):
        validate_configs(experiment, {**trace, "layers": [1]})
    with pytest.raises(ValueError, match="group_size|MXFP4"):
        validate_configs({**experiment, "quantization": {"activation": {"format": "int8_symmetric_per_row"},
                                                         "weight": {"format": "mxfp4_e2m1_ue8m0", "group_size": 16}}}, trace)
    path = tmp_path / "layer_00_q_proj.pt"
    torch.save({"sample_id": "layer_00_q_proj", "layer": 0, "projection": "q_proj",
                "activation_fp16": torch.zeros(8, 8, dtype=torch.float16), "weight_fp16": torch.zeros(8, 8, dtype=torch.float16)}, path)
    with pytest.raises(ValueError, match=r"must be \[4096,4096\]"):
        load_raw_sample(path, 0, "q_proj")
    with pytest.raises(ValueError, match="does not match its configured identity"):
        load_raw_sample(path, 6, "q_proj")
