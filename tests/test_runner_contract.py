"""CPU tests of the experiment runner: the payload contract (reference
tests/unit/test_runner_timing_contract.py), the byte formulas, the record schema and the tables,
with the native benchmark call replaced by a stub so that no GPU is needed."""

import json
from pathlib import Path

import pytest

from adangel_oyzl_b200.benchmark import runner
from adangel_oyzl_b200.ops import _sm100

ROOT = Path(__file__).resolve().parents[1]
MODE_STAGES = {
    "conversion_only": ("weight_conversion", "activation_conversion", "total"),
    "compute_only": ("gemm", "total"),
    "cold": ("weight_conversion", "activation_conversion", "gemm", "total"),
    "steady_state": ("activation_conversion", "gemm", "total"),
}


def _payload(mode, repeats=3, inner=100, variant="o0"):
    stages = [s for s in MODE_STAGES[mode] if not (variant == "o1" and s == "activation_conversion")]
    return {
        "output": object(),
        "timings_ms": {stage: [0.1 + 0.001 * i for i in range(repeats)] for stage in stages},
        "timing_method": _sm100._timing_metadata(mode, inner),
        "kernel": _sm100.kernel_metadata(variant, 128, 128, 128),
    }


@pytest.mark.parametrize("mode", list(MODE_STAGES))
def test_payload_contract_accepts_every_mode(mode):
    runner._validate_benchmark_payload(_payload(mode), 3, mode, 100)


def test_payload_contract_rejections():
    bad = _payload("cold")
    bad["timing_method"]["mode_total_timing"] = "batched_cuda_event_average"
    with pytest.raises(RuntimeError, match="wrong total timing method"):
        runner._validate_benchmark_payload(bad, 3, "cold", 100)
    with pytest.raises(RuntimeError, match="conversion_inner_repeats"):
        runner._validate_benchmark_payload(_payload("cold", inner=50), 3, "cold", 100)
    with pytest.raises(RuntimeError, match="samples, expected"):
        runner._validate_benchmark_payload(_payload("cold", repeats=2), 3, "cold", 100)
    extra = _payload("cold")
    extra["timings_ms"]["mystery"] = [1.0] * 3
    with pytest.raises(RuntimeError, match="unknown native timing stages"):
        runner._validate_benchmark_payload(extra, 3, "cold", 100)


def test_byte_and_flop_accounting():
    m = n = k = 4096
    # reference python/adangel/benchmark/runner.py:22-37
    assert runner._conversion_bytes("o0", "weight_conversion", m, n, k) == 42467328
    assert runner._conversion_bytes("o0", "activation_conversion", m, n, k) == 50348032
    assert runner._conversion_bytes("o1", "weight_conversion", m, n, k) == 25165824
    assert runner._conversion_bytes("o2", "weight_conversion", m, n, k) == 1048576
    assert runner._conversion_bytes("o2", "activation_conversion", m, n, k) == 26755072
    assert runner._fused_conversion_bytes("o2", "activation_conversion", m, n, k) == 25706496 + m * k // 32
    assert runner._conversion_bytes("o1", "activation_conversion", m, n, k) == 0
    assert runner._throughput_tflops(m, n, k, 1.0) == pytest.approx(137.438953472)


def test_shipped_configs_parse():
    import yaml

    names = sorted(p.name for p in (ROOT / "adangel_oyzl_b200" / "configs" / "experiment").glob("*.yaml"))
    assert names == ["correctness_grid.yaml", "decode_skinny.yaml", "llama7b_prefill.yaml", "o0_o1_o2_4096.yaml",
                     "sharded_large.yaml"]
    for name in names:
        cfg = yaml.safe_load((ROOT / "adangel_oyzl_b200" / "configs" / "experiment" / name).read_text())
        assert cfg["backend"]["required"] == "native" and cfg["backend"]["cuda_arch"] == "sm_100a"
        assert all(len(s) == 3 and s[2] % 64 == 0 for s in runner._shapes(cfg))
    formal = yaml.safe_load((ROOT / "adangel_oyzl_b200/configs/experiment/o0_o1_o2_4096.yaml").read_text())
    assert runner._shapes(formal) == [(4096, 4096, 4096)] and formal["timing"]["repeats"] == 200


def test_run_and_analyze_with_stubbed_native(tmp_path, monkeypatch):
    import torch
    import yaml

    from adangel_oyzl_b200.analysis import generate_report

    def fake_benchmark(inputs, variant, mode, warmup, repeats, backend="native", conversion_inner_repeats=100, formal=True, flush_l2=False):
        payload = _payload(mode, repeats, conversion_inner_repeats, variant)
        m, n, _ = inputs.shape
        payload["output"] = torch.full((m, n), {"o0": 1.0, "o1": 1.001, "o2": 1.1}[variant])
        return payload

    monkeypatch.setattr(runner, "benchmark_variant", fake_benchmark)
    monkeypatch.setattr(runner, "require_native", lambda: None)
    monkeypatch.setattr(runner, "write_environment", lambda path: Path(path).write_text("{}"))
    cfg = yaml.safe_load((ROOT / "adangel_oyzl_b200/configs/experiment/correctness_grid.yaml").read_text())
    cfg["matrix"] = {"shapes": [[64, 64, 64], [32, 96, 128]]}
    cfg["timing"].update(warmup=0, repeats=3)
    cfg_path = tmp_path / "cfg.yaml"
    cfg_path.write_text(yaml.safe_dump(cfg))
    run_dir = runner.run_experiment(cfg_path, tmp_path / "run", device="cpu")
    rows = [json.loads(line) for line in (run_dir / "results.jsonl").read_text().splitlines()]
    assert len(rows) == 2 * 4 * 3
    required = {"schema_version", "sample_id", "variant", "mode", "shape", "timings_ms", "summary",
                "equivalent_tflops", "mse_vs_o0", "kernel", "timing_method", "stable_cv", "valid"}
    for row in rows:
        assert required <= set(row) and row["schema_version"] == 2
        for stats in row["summary"].values():
            assert {"count", "mean_ms", "median_ms", "p5_ms", "p95_ms", "iqr_ms", "cv_percent", "bytes_moved",
                    "throughput_gbps"} <= set(stats)
    o2 = next(r for r in rows if r["variant"] == "o2" and r["mode"] == "compute_only")
    assert o2["mse_vs_o0"] == pytest.approx(0.01, rel=1e-4)
    with pytest.raises(FileExistsError):
        runner.run_experiment(cfg_path, tmp_path / "run", device="cpu")
    out = generate_report(run_dir, tmp_path / "report")
    for table in ("01_conversion_overhead.csv", "02_gemm_only.csv", "03_end_to_end.csv", "04_mse.csv"):
        assert (out / "tables" / table).stat().st_size > 0


def test_run_from_prepared_directory_with_stubbed_native(tmp_path, monkeypatch):
    # the runner takes its samples from a prepared directory (manifest order, hashes verified)
    import torch
    import yaml

    from adangel_oyzl_b200 import synthetic
    from adangel_oyzl_b200.trace import storage

    prepared = tmp_path / "prepared"
    records = []
    for index, shape in enumerate([(64, 64, 64), (16, 96, 128)]):
        sample = synthetic.canonical_inputs(*shape, seed=index, sample_id=f"s{index}")
        record = storage.save_prepared(sample, prepared)
        record.update(layer=index, projection="synthetic")
        records.append(record)
    storage.write_manifest(prepared, records, {"trace": {"source": "test"}}, formal=False)

    seen = []

    def fake_benchmark(inputs, variant, mode, warmup, repeats, backend="native", conversion_inner_repeats=100, formal=True, flush_l2=False):
        seen.append((inputs.sample_id, inputs.shape))
        payload = _payload(mode, repeats, conversion_inner_repeats, variant)
        payload["output"] = torch.ones((inputs.shape[0], inputs.shape[1]))
        return payload

    monkeypatch.setattr(runner, "benchmark_variant", fake_benchmark)
    monkeypatch.setattr(runner, "require_native", lambda: None)
    monkeypatch.setattr(runner, "write_environment", lambda path: Path(path).write_text("{}"))
    cfg = yaml.safe_load((ROOT / "adangel_oyzl_b200/configs/experiment/decode_skinny.yaml").read_text())
    cfg["timing"].update(warmup=0, repeats=3)
    cfg["data"]["samples"] = 1  # ignored: the prepared directory brings its own sample list
    cfg_path = tmp_path / "cfg.yaml"
    cfg_path.write_text(yaml.safe_dump(cfg))
    run_dir = runner.run_experiment(cfg_path, tmp_path / "run", device="cpu", prepared_dir=prepared)
    rows = [json.loads(line) for line in (run_dir / "results.jsonl").read_text().splitlines()]
    assert {(r["sample_id"], tuple(r["shape"])) for r in rows} == {("s0", (64, 64, 64)), ("s1", (16, 96, 128))}
    assert set(seen) == {("s0", (64, 64, 64)), ("s1", (16, 96, 128))}
    # decode-shaped GEMMs carry their weight-streaming byte count
    decode = next(r for r in rows if r["sample_id"] == "s1" and r["variant"] == "o2" and r["mode"] == "compute_only")
    assert decode["summary"]["gemm"]["bytes_moved"] == 96 * 128 // 2 + 96 * 4 + 16 * 128 // 2 + 16 * 4 + 4 * 16 * 96
    # a corrupted sample file is refused
    victim = prepared / "s0.pt"
    victim.write_bytes(victim.read_bytes() + b"x")
    with pytest.raises(ValueError, match="SHA-256 does not match"):
        runner.run_experiment(cfg_path, tmp_path / "run2", device="cpu", prepared_dir=prepared)
