"""Wrappers of the native device kernels."""
