"""fairring_b200: a reduction-server all-reduce backend for PyTorch on B200.

``import fairring_b200`` (or the drop-in alias ``import fairring``) registers
the ``"fairring"`` backend with ``torch.distributed``; after that

    torch.distributed.init_process_group("fairring")

gives a process group whose all_reduce / reduce_scatter / all_gather run on
hand-written sm_100a kernels over peer-mapped NVLink memory (CUDA tensors) or
on POSIX shared memory (CPU tensors), and whose other collectives go to NCCL or
Gloo.  Counterpart of ``fairring/__init__.py`` in the reference
(fairring/__init__.py:17-49): same backend name, same environment variables,
same non-extended factory signature ``(store, rank, size, timeout)``.

Environment variables (read when a process group is created):

=============================  ==========================================================
FAIRRING_TOTAL_MEMORY          staging bytes per GPU (default 50 MiB, notice on stderr)
FAIRRING_PADDING_MEMORY        accepted for compatibility; tails are predicated in-kernel
FAIRRING_PARALLELISM           slices in flight = side streams/channels (default 16, clamped
                               so that half a channel slot stays >= 4 MiB)
FAIRRING_SLICE_SIZE            max bytes per slice (default 25 MiB, DDP's bucket size)
FAIRRING_GPUS_PER_MACHINE      D of the M x D grouping (default: all ranks of a host)
FAIRRING_RANK_LAYOUT           "standard" (rank = m*D+d) or "favorable" (rank = d*M+m)
FAIRRING_ALGO                  auto | ll | oneshot | twoshot | hier | nvls | nvls_oneshot | pipe
FAIRRING_BLOCKS                thread blocks per kernel (default 16, max 64)
FAIRRING_SM_BUDGET             SMs the collectives may occupy at once (default 64): the number
                               of channels is at most SM_BUDGET / BLOCKS.  Raise it (up to the
                               SM count) for stand-alone all-reduce bandwidth, keep it low to
                               leave the GPU to backward
FAIRRING_LL_MAX                largest message (bytes) for the flag-in-data kernel (default 32 KiB;
                               0 turns it off); FAIRRING_LL_CHANNELS channels carry its areas
FAIRRING_LL2_MAX               largest message (bytes) for its two-shot form (default 1 MiB; the
                               areas shrink it when the memory budget is small)
FAIRRING_INLINE_SMALL          1 (default): a blocking all_reduce that fits that kernel runs on the
                               caller's own stream
FAIRRING_ONESHOT_MAX           largest message (bytes) for the one-shot kernel
FAIRRING_DIRECT_BLOCKS         thread blocks of an in-place launch on symmetric memory (0: FAIRRING_BLOCKS)
FAIRRING_DIRECT_UNROLL         16-byte multimem loads a thread keeps in flight in the in-place kernel
FAIRRING_NVLS                  auto | on | off   (NVSwitch multicast kernels)
FAIRRING_NVLS_MIN              smallest message (bytes) for the NVLS two-shot kernel
FAIRRING_NVLS_ONESHOT_MAX      largest message (bytes) for the NVLS one-shot kernel
FAIRRING_TRANSPORT             auto | vmm | ipc  (how peer memory is shared)
FAIRRING_DIRECT                auto | nvls | p2p | off  (in-place kernels for tensors from
                               ``symmetric_empty``: no staging copies)
FAIRRING_PIPE                  auto | on | off: ordinary tensors of FAIRRING_PIPE_MIN bytes and more
                               take the pipelined kernel (bulk copy in, switch reduce, bulk copy
                               out, chunk by chunk in one launch); its staging rings take a third
                               of the memory budget
FAIRRING_PIPE_MIN              smallest message (bytes) for the pipelined kernel (default 64 MiB; it
                               also needs ring slots of 4 MiB or more, i.e. a memory budget of
                               about 100 MiB, below which the staged kernels serve)
FAIRRING_PIPE_BLOCKS           thread blocks of a pipelined launch (default 16)
FAIRRING_PIPE_CHANNELS         rings, i.e. pipelined launches that may overlap (default 2)
FAIRRING_PIPE_SLOTS            ring length in chunks (default 4)
FAIRRING_PIPE_CHUNK            chunk bytes (default: 16 MiB or the ring slot, whichever is smaller)
FAIRRING_PIPE_STAGE / _STAGES  shared-memory stage bytes / stages per copy role (16 KiB x 6)
FAIRRING_DIRECT_MAX_SLICES     in-place NVLS messages are split over at most this many channels
FAIRRING_DIRECT_MIN_SLICE      ... down to slices of this many bytes
FAIRRING_DEVICE_TIMEOUT_MS     limit of one device-side wait on a peer (default: the process
                               group's timeout; a wait that runs out leaves the tensor
                               unreduced and poisons the engine until reset())
FAIRRING_TUNING_TABLE          path of the measured thresholds (default: tuning.json beside this
                               file, keyed by world size); "off" ignores it
FAIRRING_COMMAND_THREAD        1: enqueue kernels from a dedicated thread
FAIRRING_BLOCKING_WAIT         1: Work.wait() blocks the host and reports kernel failures
=============================  ==========================================================
"""

from __future__ import annotations

import importlib.util
import os
import sys
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist

__version__ = "0.1.0"

_HERE = Path(__file__).resolve().parent


def _load_native():
    from . import _build

    so = _HERE / "_C.so"
    if not so.exists():
        # First use in a fresh checkout: compile in-tree (minutes, once).
        sys.stderr.write("fairring_b200: building the native module (first use)...\n")
        _build.build()
    spec = importlib.util.spec_from_file_location("fairring_b200._C", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["fairring_b200._C"] = mod
    return mod


_C = _load_native()

DEFAULT_TOTAL_MEMORY = 50 * 1024 * 1024
DEFAULT_PADDING_MEMORY = 1024 * 1024
DEFAULT_PARALLELISM = 16
DEFAULT_SLICE_SIZE = 25 * 1024 * 1024


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ[name])
    except KeyError:
        return default


# Option name -> the environment variable that overrides it.
_TUNABLES = {
    "ll_max_bytes": "FAIRRING_LL_MAX",
    "ll2_max_bytes": "FAIRRING_LL2_MAX",
    "oneshot_max_bytes": "FAIRRING_ONESHOT_MAX",
    "nvls_oneshot_max_bytes": "FAIRRING_NVLS_ONESHOT_MAX",
    "pipe_min_bytes": "FAIRRING_PIPE_MIN",
    "pipe_blocks": "FAIRRING_PIPE_BLOCKS",
    "pipe_chunk_bytes": "FAIRRING_PIPE_CHUNK",
    "blocks": "FAIRRING_BLOCKS",
    "direct_max_slices": "FAIRRING_DIRECT_MAX_SLICES",
    "direct_unroll": "FAIRRING_DIRECT_UNROLL",
    "direct_blocks": "FAIRRING_DIRECT_BLOCKS",
}


def tuning_table(world: int) -> dict:
    """Measured thresholds for this world size from ``tuning.json`` next to this
    file (written by ``python -m fairring_b200.bench.tune --write-table``), or
    an empty dict.  ``FAIRRING_TUNING_TABLE=off`` ignores the file; a path
    names another file."""
    where = os.environ.get("FAIRRING_TUNING_TABLE", "")
    if where.lower() == "off":
        return {}
    path = Path(where) if where else _HERE / "tuning.json"
    try:
        import json

        table = json.loads(path.read_text()).get(str(world), {})
    except (OSError, ValueError):
        return {}
    return {k: int(v) for k, v in table.items() if k in _TUNABLES}


def options_from_env(timeout: timedelta | None = None, world: int = 0) -> "_C.Options":
    """Build backend options: defaults, then the measured table for this world
    size, then the FAIRRING_* environment variables."""
    opts = _C.Options(timeout) if timeout is not None else _C.Options()
    for key, value in tuning_table(world).items():
        if _TUNABLES[key] not in os.environ:
            setattr(opts, key, value)
    if "FAIRRING_TOTAL_MEMORY" not in os.environ:
        sys.stderr.write(
            "The Fairring process group will allocate up to 50 MiB of staging memory "
            "on each GPU. This can be tuned by setting the FAIRRING_TOTAL_MEMORY "
            "environment variable (to an amount of bytes).\n"
        )
    opts.max_memory_allocated_in_bytes = _env_int("FAIRRING_TOTAL_MEMORY", DEFAULT_TOTAL_MEMORY)
    opts.max_padding_allocated_in_bytes = _env_int("FAIRRING_PADDING_MEMORY", DEFAULT_PADDING_MEMORY)
    opts.min_parallelism = _env_int("FAIRRING_PARALLELISM", DEFAULT_PARALLELISM)
    opts.slice_size_in_bytes = _env_int("FAIRRING_SLICE_SIZE", DEFAULT_SLICE_SIZE)
    opts.is_high_priority_stream = True
    opts.gpus_per_machine = _env_int("FAIRRING_GPUS_PER_MACHINE", 0)
    layout = os.environ.get("FAIRRING_RANK_LAYOUT", "standard").lower()
    if layout not in ("standard", "favorable"):
        raise ValueError("FAIRRING_RANK_LAYOUT must be 'standard' or 'favorable'")
    opts.favorable_layout = layout == "favorable"
    opts.algo = os.environ.get("FAIRRING_ALGO", "auto").lower()
    opts.blocks = _env_int("FAIRRING_BLOCKS", opts.blocks)
    opts.sm_budget = _env_int("FAIRRING_SM_BUDGET", opts.sm_budget)
    opts.oneshot_max_bytes = _env_int("FAIRRING_ONESHOT_MAX", opts.oneshot_max_bytes)
    opts.ll_max_bytes = _env_int("FAIRRING_LL_MAX", opts.ll_max_bytes)
    opts.ll2_max_bytes = _env_int("FAIRRING_LL2_MAX", opts.ll2_max_bytes)
    opts.ll_channels = _env_int("FAIRRING_LL_CHANNELS", opts.ll_channels)
    opts.inline_small = os.environ.get("FAIRRING_INLINE_SMALL", "1") == "1"
    opts.direct_unroll = _env_int("FAIRRING_DIRECT_UNROLL", opts.direct_unroll)
    opts.direct_blocks = _env_int("FAIRRING_DIRECT_BLOCKS", opts.direct_blocks)
    opts.nvls_min_bytes = _env_int("FAIRRING_NVLS_MIN", opts.nvls_min_bytes)
    opts.nvls_oneshot_max_bytes = _env_int("FAIRRING_NVLS_ONESHOT_MAX", opts.nvls_oneshot_max_bytes)
    opts.device_timeout_ms = _env_int("FAIRRING_DEVICE_TIMEOUT_MS", opts.device_timeout_ms)
    opts.nvls = os.environ.get("FAIRRING_NVLS", "auto").lower()
    opts.transport = os.environ.get("FAIRRING_TRANSPORT", "auto").lower()
    opts.direct = os.environ.get("FAIRRING_DIRECT", "auto").lower()
    opts.pipe = os.environ.get("FAIRRING_PIPE", "auto").lower()
    opts.pipe_min_bytes = _env_int("FAIRRING_PIPE_MIN", opts.pipe_min_bytes)
    opts.pipe_blocks = _env_int("FAIRRING_PIPE_BLOCKS", opts.pipe_blocks)
    opts.pipe_channels = _env_int("FAIRRING_PIPE_CHANNELS", opts.pipe_channels)
    opts.pipe_slots = _env_int("FAIRRING_PIPE_SLOTS", opts.pipe_slots)
    opts.pipe_chunk_bytes = _env_int("FAIRRING_PIPE_CHUNK", opts.pipe_chunk_bytes)
    opts.pipe_stage_bytes = _env_int("FAIRRING_PIPE_STAGE", opts.pipe_stage_bytes)
    opts.pipe_stages = _env_int("FAIRRING_PIPE_STAGES", opts.pipe_stages)
    opts.direct_max_slices = _env_int("FAIRRING_DIRECT_MAX_SLICES", opts.direct_max_slices)
    opts.direct_min_slice_bytes = _env_int("FAIRRING_DIRECT_MIN_SLICE", opts.direct_min_slice_bytes)
    opts.command_thread = os.environ.get("FAIRRING_COMMAND_THREAD", "0") == "1"
    opts.blocking_wait = os.environ.get("FAIRRING_BLOCKING_WAIT", "0") == "1"
    opts.boot_id_override = os.environ.get("FAIRRING_BOOT_ID", "")
    return opts


def _delegate_factory(store, rank: int, size: int, timeout: timedelta):
    """Lazily build the library backend that serves what this one delegates."""

    def make(kind: str):
        if kind == "cuda":
            pg_opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
            pg_opts._timeout = timeout
            return dist.ProcessGroupNCCL(dist.PrefixStore("nccl", store), rank, size, pg_opts)
        return dist.ProcessGroupGloo(dist.PrefixStore("gloo", store), rank, size, timeout=timeout)

    return make


def create_process_group_fairring(store, rank, size, timeout):
    """Factory registered with torch.distributed (fairring/__init__.py:17-46 in the reference)."""
    backend = _C.Backend(store, rank, size, options_from_env(timeout, world=size))
    backend.set_delegate_factory(_delegate_factory(store, rank, size, timeout))
    return backend


def _register() -> None:
    if "FAIRRING" in dist.Backend._plugins:
        return
    dist.Backend.register_backend(
        "fairring", create_process_group_fairring, extended_api=False, devices=["cpu", "cuda"]
    )


_register()


def get_backend(group=None, device: str | torch.device | None = None):
    """The native backend object behind a process group (for the extra methods:
    ``allreduce_fused``, ``stats``, ``describe``, ``check_health``, ``reset``)."""
    group = group if group is not None else dist.group.WORLD
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    return group._get_backend(torch.device(device))


def launch_count() -> int:
    """Kernels launched by this library in this process so far."""
    return int(_C.launch_count())


__all__ = [
    "create_process_group_fairring",
    "options_from_env",
    "get_backend",
    "launch_count",
    "_C",
]
