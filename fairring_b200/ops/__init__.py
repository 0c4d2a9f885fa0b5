"""Fused single-GPU ops used by the training drivers."""

from .optim import FlatAdamW  # noqa: F401
