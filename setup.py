"""Packaging for fairring_b200.

    python setup.py build_ext --inplace     # compile fairring_b200/_C.so in the tree
    pip install --no-build-isolation .       # install both packages (fairring, fairring_b200)

The native module is built by ``fairring_b200/_build.py`` for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``); there is no other target.
Counterpart of the reference's setup.py (setup.py:53-98).  The reference's
NCCL linkage switches (static / USE_SYSTEM_NCCL / USE_TORCH_NCCL, setup.py:33-50
and version.map) have no equivalent: this library does not link NCCL at all, it
reaches NCCL only through torch's ProcessGroupNCCL for the delegated collectives.
``FAIRRING_VERSION`` overrides the version string, as in the reference.
"""

import os
import subprocess
import sys
from pathlib import Path

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


def version() -> str:
    v = os.environ.get("FAIRRING_VERSION")
    if v:
        return v
    base = "0.1.0"
    try:
        h = subprocess.check_output(["git", "rev-parse", "--short", "HEAD"], cwd=ROOT,
                                    stderr=subprocess.DEVNULL).decode().strip()
        dirty = subprocess.call(["git", "diff", "--quiet"], cwd=ROOT) != 0
        return f"{base}+git{h}" + (".dirty" if dirty else "")
    except Exception:
        return base


def _build_native():
    sys.path.insert(0, str(ROOT))
    from fairring_b200 import _build

    _build.build()


class BuildExt(Command):
    description = "compile fairring_b200/_C.so in the source tree"
    user_options = [("inplace", "i", "always in place")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


setup(
    name="fairring-b200",
    version=version(),
    description="Reduction-server all-reduce backend for PyTorch on B200 (sm_100a kernels over NVLink 5 / NVSwitch)",
    packages=find_packages(include=["fairring", "fairring_b200", "fairring_b200.*"]),
    package_data={"fairring_b200": ["_C.so", "csrc/*", "csrc/kernels/*"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6"],
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
    entry_points={"console_scripts": [
        "fairring-launch-benchmark=fairring_b200.bench.launch:main",
        "fairring-sweep=fairring_b200.bench.sweep:main",
    ]},
)
