"""Device-side timing: CUDA events on the launching stream, max over ranks."""

from __future__ import annotations

import torch
import torch.distributed as dist


def device_time_ms(fn, iters: int, warmup: int = 3, flush_l2: bool = False) -> float:
    """Average milliseconds per call of ``fn`` over ``iters`` calls, after
    ``warmup`` untimed calls.  With ``flush_l2`` a 256 MiB buffer is rewritten
    before every timed call (excluded from the time by timing calls one by one)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if not flush_l2:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    total = 0.0
    for _ in range(iters):
        scratch.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def max_over_ranks(value: float, device=None) -> float:
    """The slowest rank's value (what a collective's time is)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device or "cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
