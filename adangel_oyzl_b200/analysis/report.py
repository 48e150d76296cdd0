"""The four contract tables of one completed run (``tables/01..04*.csv``).

Same tables as ``python/adangel/analysis/report.py:20-102`` of the reference, keyed additionally by
shape because a run here may cover several shapes; the MSE summary rows carry the reference's
bootstrap confidence interval of the median (parameters from the run's ``config.yaml``).  Every table
row keeps its ``cv_percent``.  The reference's four figures need matplotlib; they are drawn only when it
is installed.
"""

from __future__ import annotations

import json
from pathlib import Path

from ..benchmark.metrics import bootstrap_median_ci


def _records(run_dir: Path, allow_unstable: bool) -> list[dict]:
    rows = [json.loads(line) for line in (run_dir / "results.jsonl").read_text(encoding="utf-8").splitlines() if line]
    if not rows:
        raise RuntimeError("run is empty")
    if not allow_unstable and any(not row["valid"] for row in rows):
        raise RuntimeError("run contains invalid/CV-failed records")
    return rows


def generate_report(run_dir, output_dir, allow_unstable: bool = False) -> Path:
    import pandas as pd

    run_dir, output_dir = Path(run_dir), Path(output_dir)
    table_dir = output_dir / "tables"
    table_dir.mkdir(parents=True, exist_ok=True)
    records = _records(run_dir, allow_unstable)
    import yaml

    config_path = run_dir / "config.yaml"
    config = yaml.safe_load(config_path.read_text(encoding="utf-8")) if config_path.exists() else {}
    statistics_cfg = config.get("statistics") or {}
    bootstrap_samples = int(statistics_cfg.get("bootstrap_samples", 2000))
    confidence = float(statistics_cfg.get("confidence", 0.95))
    seed = int((config.get("experiment") or {}).get("seed", 0))

    flat = []
    for row in records:
        base = {k: row[k] for k in ("sample_id", "variant", "mode", "mse_vs_o0", "equivalent_tflops")}
        base["shape"] = "x".join(str(x) for x in row["shape"])
        for stage, stats in row["summary"].items():
            flat.append({**base, "stage": stage, **stats})
    frame = pd.DataFrame(flat)

    conversion_names = {"o0": ["weight_conversion", "activation_conversion"], "o1": ["weight_conversion"],
                        "o1x": ["weight_conversion"], "o2": ["weight_conversion", "activation_conversion"]}
    conv = frame[frame["mode"].eq("conversion_only")].copy()
    conv = conv[conv.apply(lambda r: r["stage"] in conversion_names.get(r["variant"], []), axis=1)]
    conv.to_csv(table_dir / "01_conversion_overhead.csv", index=False)

    gemm = frame[(frame["mode"] == "compute_only") & (frame["stage"] == "gemm")].copy()
    baseline = gemm[gemm["variant"] == "o0"][["sample_id", "median_ms"]].rename(columns={"median_ms": "o0_median_ms"})
    if len(baseline):
        gemm = gemm.merge(baseline, on="sample_id", how="left")
        gemm["speedup_vs_o0"] = gemm["o0_median_ms"] / gemm["median_ms"]
    gemm.to_csv(table_dir / "02_gemm_only.csv", index=False)

    stages = ["weight_conversion", "activation_conversion", "gemm", "total"]
    e2e = frame[(frame["mode"].isin(["cold", "steady_state"])) & (frame["stage"].isin(stages))]
    e2e.to_csv(table_dir / "03_end_to_end.csv", index=False)

    mse_rows = {(r["sample_id"], r["variant"]): r["mse_vs_o0"] for r in records if r["mode"] == "compute_only"}
    mse_frame = pd.DataFrame([{"sample_id": s, "variant": v, "mse_vs_o0": x} for (s, v), x in mse_rows.items()])
    summary = []
    if len(mse_frame):
        for variant, group in mse_frame.groupby("variant"):
            values = [float(v) for v in group["mse_vs_o0"].tolist() if v is not None and v == v]
            low, high = bootstrap_median_ci(values, bootstrap_samples, confidence, seed) if values else (None, None)
            summary.append({"sample_id": "__summary__", "variant": variant, "mse_vs_o0": group["mse_vs_o0"].median(),
                            "iqr": group["mse_vs_o0"].quantile(0.75) - group["mse_vs_o0"].quantile(0.25),
                            "max": group["mse_vs_o0"].max(), "bootstrap_median_ci_low": low,
                            "bootstrap_median_ci_high": high})
    pd.concat([mse_frame, pd.DataFrame(summary)], ignore_index=True).to_csv(table_dir / "04_mse.csv", index=False)

    try:
        import matplotlib
    except ImportError:
        return output_dir
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    figure_dir = output_dir / "figures"
    figure_dir.mkdir(parents=True, exist_ok=True)
    if len(gemm):
        ax = gemm.groupby("variant")["equivalent_tflops"].median().plot.bar()
        ax.set_ylabel("Equivalent throughput (TFLOP/s)")
        ax.figure.tight_layout()
        ax.figure.savefig(figure_dir / "02_gemm_only.png", dpi=180)
        plt.close(ax.figure)
    return output_dir
