"""Benchmark tooling: kernel micro-benchmarks with roofline fractions and the evidence harness."""
