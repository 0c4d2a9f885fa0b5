"""Synthetic-data training workloads used to measure the backend under DDP."""

from .decoder import DecoderConfig, DecoderLM  # noqa: F401
from .encoder import EncoderConfig, EncoderMLM, mask_tokens  # noqa: F401
from .resnet import ResNet50  # noqa: F401
