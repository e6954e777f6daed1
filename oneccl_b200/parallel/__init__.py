"""Parallelism building blocks built on the communicator."""
