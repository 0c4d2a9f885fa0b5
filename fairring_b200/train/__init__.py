"""Data-parallel training drivers on synthetic data (decoder LM, ResNet-50, RoBERTa-style encoder)."""
