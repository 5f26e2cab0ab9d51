"""Benchmark drivers (command line compatible with the reference's benchmarks/*.py)."""
