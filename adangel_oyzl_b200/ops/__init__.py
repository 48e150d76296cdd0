from .dispatch import benchmark_variant, run_o0, run_o1, run_o1x, run_o2

__all__ = ["run_o0", "run_o1", "run_o2", "run_o1x", "benchmark_variant"]
