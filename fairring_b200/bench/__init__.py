"""Micro-benchmarks: all-reduce sweep and the bucket benchmark launcher."""
