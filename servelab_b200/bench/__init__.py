"""Measurements: kernel microbenchmarks (``python -m servelab_b200.bench.kernel_bench``)."""
