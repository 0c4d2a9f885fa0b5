"""In-tree build of the native module ``fairring_b200._C``.

The sources under ``csrc/`` are compiled for sm_100a only and linked into
``fairring_b200/_C.so`` next to this file, so that the built module travels
with the source tree (no JIT cache, nothing installed into site-packages).
Counterpart of the reference's setup.py (setup.py:53-98), which builds a
``CUDAExtension`` of host-only C++; here the same job also compiles the
hand-written kernels.
"""

from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_CSRC = _HERE / "csrc"
_SO = _HERE / "_C.so"
_BUILD_DIR = _HERE / "build"

SOURCES = [
    "bindings.cpp",
    "backend.cpp",
    "engine.cpp",
    "symmem.cpp",
    "topology.cpp",
    "cpu_path.cpp",
    "emulate.cpp",
    "bench_client.cpp",
    "local_ops.cpp",
    "selftest.cpp",
    "kernels/collectives.cu",
    "kernels/collectives_u8.cu",
    "kernels/collectives_i8.cu",
    "kernels/collectives_i32.cu",
    "kernels/collectives_i64.cu",
    "kernels/collectives_f16.cu",
    "kernels/collectives_bf16.cu",
    "kernels/collectives_f32.cu",
    "kernels/collectives_f64.cu",
    "kernels/collectives_f32_bf16.cu",
    "kernels/collectives_f32_f16.cu",
    "kernels/local_ops.cu",
    "kernels/layernorm.cu",
    "kernels/cross_entropy.cu",
    "kernels/noalloc_allreduce.cu",
    "kernels/pipe_allreduce.cu",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-g1", "-Wno-unused-variable"]


def _shared_libstdcxx_flags() -> list[str]:
    """Make sure the module links the shared libstdc++.

    Some toolchain wrappers resolve ``-lstdc++`` to a static archive; a private
    copy of the C++ runtime inside the module clashes with the one torch uses
    (iostreams crash on first use).  Put a directory with a real
    ``libstdc++.so`` first on the search path.
    """
    import glob

    for d in sorted(glob.glob("/usr/lib/gcc/x86_64-linux-gnu/*"), reverse=True):
        so = os.path.join(d, "libstdc++.so")
        if os.path.exists(so):  # follows the symlink: must not dangle
            return [f"-L{d}"]
    return []


def sources() -> list[str]:
    return [str(_CSRC / s) for s in SOURCES if (_CSRC / s).exists()]


def _newest_source_mtime() -> float:
    newest = 0.0
    for p in _CSRC.rglob("*"):
        if p.suffix in {".cpp", ".cu", ".h", ".cuh"}:
            newest = max(newest, p.stat().st_mtime)
    return newest


def is_built() -> bool:
    return _SO.exists()


def is_stale() -> bool:
    return not _SO.exists() or _SO.stat().st_mtime < _newest_source_mtime()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if needed) and return the path of ``_C.so``."""
    if _SO.exists() and not force and not is_stale():
        return _SO
    import torch  # noqa: F401  (must be imported before cpp_extension)
    from torch.utils import cpp_extension

    _BUILD_DIR.mkdir(exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
    cpp_extension.load(
        name="_C",
        sources=sources(),
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=NVCC_FLAGS,
        extra_ldflags=_shared_libstdcxx_flags() + ["-lrt"],
        extra_include_paths=[str(_CSRC)],
        build_directory=str(_BUILD_DIR),
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    built = _BUILD_DIR / "_C.so"
    if not built.exists():
        raise RuntimeError(f"build finished but {built} is missing")
    tmp = _SO.with_suffix(".so.tmp")
    shutil.copy2(built, tmp)
    os.replace(tmp, _SO)
    return _SO


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
