"""Benchmark harnesses that ship with the package (kernel micro-benchmarks,
per-layer DP step timings, step profiles)."""
