"""Benchmark drivers (collective sweep, GEMM, tensor-parallel MLP, MoE)."""
