"""Host code under a thread sanitizer: the command queue (several producers,
one consumer) and the shared-memory host path with threads playing the ranks.
A test on results alone would not see a data race; TSAN does."""

import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "fairring_b200" / "csrc"


def test_host_code_under_thread_sanitizer(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    import torch

    inc = Path(torch.__file__).resolve().parent / "include"
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    exe = tmp_path / "selftest_tsan"
    cmd = [gxx, "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-DFR_SELFTEST_STANDALONE",
           f"-I{CSRC}", f"-I{inc}", f"-I{cuda_inc}",
           str(CSRC / "selftest.cpp"), str(CSRC / "cpu_path.cpp"), "-o", str(exe), "-pthread", "-lrt"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "tsan" in build.stderr.lower() and "cannot find" in build.stderr.lower():
        pytest.skip("libtsan is not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 second_deadlock_stack=1")
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    sys.stdout.write(run.stdout)
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-3000:]
    assert run.returncode == 0, run.stderr[-2000:]
