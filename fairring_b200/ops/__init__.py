"""Fused single-GPU ops used by the training drivers."""

from .optim import FlatAdamW  # noqa: F401
from .layernorm import FusedLayerNorm, add_layer_norm, fused_layer_norm  # noqa: F401
from .cross_entropy import fused_cross_entropy  # noqa: F401
