"""The experiment runner, the four report tables and the acceptance check, on the device.

The reference drives these from its CLI on the target GPU (``python -m adangel run / analyze`` and
``scripts/validate_o{0,1,2}.py``); here a small shape keeps the run to seconds while going through the same
code: native benchmark calls in every mode, payload validation, JSONL schema 2, CV statistics, MSE against O0
and the bootstrap interval of its median.
"""

import json

import numpy as np
import pytest
import yaml

from oracle import adangel_oracle as orc

pytestmark = pytest.mark.gpu


def _config(tmp_path, variants):
    cfg = {
        "experiment": {"name": "runner_smoke", "seed": 20250805, "formal": False},
        "matrix": {"shapes": [[256, 384, 512], [48, 256, 256]]},
        "data": {"source": "synthetic_canonical", "samples": 2},
        "variants": variants,
        "modes": ["conversion_only", "compute_only", "cold", "steady_state"],
        "timing": {"warmup": 2, "repeats": 5, "conversion_inner_repeats": 4, "max_cv_percent": 1000.0},
        "statistics": {"bootstrap_samples": 200, "confidence": 0.9},
        "backend": {"required": "native", "cuda_arch": "sm_100a"},
    }
    path = tmp_path / "config.yaml"
    path.write_text(yaml.safe_dump(cfg), encoding="utf-8")
    return path


def test_run_and_analyze_on_the_device(tmp_path):
    import pandas as pd

    from adangel_oyzl_b200.analysis import generate_report
    from adangel_oyzl_b200.benchmark.runner import run_experiment

    run_dir = run_experiment(_config(tmp_path, ["o0", "o1", "o2", "o1x"]), tmp_path / "run")
    rows = [json.loads(line) for line in (run_dir / "results.jsonl").read_text().splitlines()]
    assert len(rows) == 2 * 2 * 4 * 4  # shapes x samples x modes x variants
    for row in rows:
        assert row["schema_version"] == 2 and row["valid"] is True
        assert set(row["timings_ms"]) <= {"weight_conversion", "activation_conversion", "gemm", "total"}
        assert all(len(v) == 5 for v in row["timings_ms"].values())
        assert row["kernel"]["mma_family"].startswith("tcgen05.mma")
        if row["variant"] in ("o1", "o1x"):
            assert "activation_conversion" not in row["timings_ms"]  # the reference's O1 stage sets
    # the MSE recorded for a sample is the oracle's, within 2 %
    sample = next(r for r in rows if r["mode"] == "compute_only" and r["variant"] == "o2" and r["shape"] == [256, 384, 512])
    args = orc.canonical_inputs(256, 384, 512, seed=20250805 + int(sample["sample_id"][-2:]))
    o0, o2 = orc.run_o0(*args)["output"], orc.run_o2(*args)["output"]
    assert sample["mse_vs_o0"] == pytest.approx(orc.mse_fp64(o2, o0), rel=0.02)
    report = generate_report(run_dir, tmp_path / "report")
    for name in ("01_conversion_overhead.csv", "02_gemm_only.csv", "03_end_to_end.csv", "04_mse.csv"):
        assert (report / "tables" / name).exists()
    mse = pd.read_csv(report / "tables" / "04_mse.csv")
    summary = mse[mse["sample_id"] == "__summary__"].set_index("variant")
    assert summary.loc["o0", "mse_vs_o0"] == 0.0
    for variant in ("o1", "o2", "o1x"):
        assert summary.loc[variant, "bootstrap_median_ci_low"] <= summary.loc[variant, "mse_vs_o0"] <= summary.loc[variant, "bootstrap_median_ci_high"]
    assert "cv_percent" in pd.read_csv(report / "tables" / "02_gemm_only.csv").columns
    conv = pd.read_csv(report / "tables" / "01_conversion_overhead.csv")
    assert set(conv[conv["variant"] == "o1"]["stage"]) == {"weight_conversion"}


@pytest.mark.parametrize("variant", ["o0", "o1", "o2", "o1x"])
def test_acceptance_check(variant):
    import torch

    from adangel_oyzl_b200.synthetic import canonical_inputs
    from adangel_oyzl_b200.validate import validate_variant

    inputs = canonical_inputs(320, 384, 512, seed=77, device="cuda")
    host = tuple(t.cpu().numpy() for t in (inputs.A_int8, inputs.A_scale, inputs.W_mxfp4, inputs.W_scale))
    expected = {"o0": orc.run_o0, "o1": orc.run_o1, "o2": orc.run_o2, "o1x": orc.run_o1x}[variant](*host)["output"]
    report = validate_variant(variant, inputs, warmup=1, repeats=3, conversion_inner_repeats=2,
                              expected_output=torch.from_numpy(np.ascontiguousarray(expected)))
    assert report["passed"], report["violations"]
    assert report["performance_gate"]["applied"] is False
    assert report["max_abs_error"] <= 1e-3
