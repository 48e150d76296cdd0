from .metrics import mse_fp64, percentile, summarize_samples

__all__ = ["mse_fp64", "percentile", "summarize_samples"]
