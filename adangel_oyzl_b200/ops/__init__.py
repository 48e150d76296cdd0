from .dispatch import benchmark_variant, run_o0, run_o1, run_o2

__all__ = ["run_o0", "run_o1", "run_o2", "benchmark_variant"]
