"""Benchmark models."""
