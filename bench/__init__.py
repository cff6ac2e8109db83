"""Benchmark helpers: per-kernel roofline microbenchmarks and serving workloads."""
