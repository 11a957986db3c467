"""Device-timed micro-benchmarks of individual kernels (``python -m incin_b200.benchmarks.kernels``)."""
