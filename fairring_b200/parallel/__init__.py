"""Data-parallel wrappers and DDP communication hooks for the fairring backend."""

from .ddp import FlatDataParallel, FusedHookState, fused_allreduce_hook  # noqa: F401
