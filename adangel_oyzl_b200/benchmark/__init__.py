from .metrics import bootstrap_median_ci, mse_fp64, percentile, summarize_samples

__all__ = ["bootstrap_median_ci", "mse_fp64", "percentile", "summarize_samples"]
