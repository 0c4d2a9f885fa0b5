"""Synthetic-data training workloads used to measure the backend under DDP."""

from .decoder import DecoderConfig, DecoderLM  # noqa: F401
